"""Environment of the MARFT code workflow: the Actor's program is run against the task's test cases."""
from siirl_b200.utils.reward_score import prime_code


class CodeEnv:
    def reset(self):
        pass

    def step(self, actions, ground_truth):
        score = prime_code.compute_score(actions[-1], ground_truth, continuous=True)
        score = float(score["score"] if isinstance(score, dict) else score)
        solved = score >= 1.0
        verdict = "All tests pass." if solved else f"Tests passed: {score:.0%}. Fix the program."
        return [f"previous program: {act}\n{verdict}" for act in actions], score, solved
