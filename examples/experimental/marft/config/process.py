"""Per-agent prompt hooks of the two-agent (Reasoner -> Actor) MARFT workflow.

``pre_process(tokenizer, prompt_id, obs, **kwargs) -> List[int]`` builds the token ids an agent is prompted with from
the running conversation (``prompt_id``: the task plus what the agents before it wrote in this turn) and the
environment's verdict on the previous turn (``obs``, ``None`` in the first turn).  ``kwargs`` are the node's
``pre_process_kwargs``; ``pre_chat_template`` may use ``${prompt}`` and ``${obs}``.

``post_process(tokenizer, prompt_id, response_id, **kwargs) -> List[int]`` joins the agent's response to the
conversation; ``post_chat_template`` is the text put between them (the speaker tag)."""
from string import Template


def pre_process(tokenizer, prompt_id, obs, **kwargs):
    template = kwargs.get("pre_chat_template")
    text = tokenizer.decode(prompt_id, skip_special_tokens=True)
    if template:
        text = Template(template).safe_substitute(prompt=text, obs=obs or "")
    elif obs:
        text = f"{text}\n{obs}"
    if kwargs.get("use_chat_template", False) and getattr(tokenizer, "chat_template", None):
        return list(tokenizer.apply_chat_template([{"role": "user", "content": text}], tokenize=True,
                                                  add_generation_prompt=True))
    return list(tokenizer.encode(text, add_special_tokens=False))


def post_process(tokenizer, prompt_id, response_id, **kwargs):
    tag = kwargs.get("post_chat_template") or ""
    tag_ids = list(tokenizer.encode(tag, add_special_tokens=False)) if tag else []
    return list(prompt_id) + tag_ids + list(response_id)
