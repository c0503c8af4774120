"""Environment of the MARFT math workflow: one instance per sample, judged after every turn.

``step(actions, ground_truth)`` receives what each agent wrote in the turn (in agent order; the last entry is the
Actor's answer) and returns ``(next_obs, score, should_stop)``: the observation shown to each agent in the next turn,
the turn's reward, and whether the sample is finished."""
from siirl_b200.utils.reward_score.math import compute_score


class MathEnv:
    def __init__(self):
        self.turns = 0

    def reset(self):
        self.turns = 0

    def step(self, actions, ground_truth):
        self.turns += 1
        score = float(compute_score(actions[-1], str(ground_truth)))
        solved = score >= 1.0
        verdict = "This answer is right." if solved else "This answer is wrong. Reflect on the mistake and try again."
        next_obs = [f"previous attempt: {act}\n{verdict}" for act in actions]
        return next_obs, score, solved
