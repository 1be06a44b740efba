"""Gemma-4 chat templates of the serve surface (crates/ksearch_gguf/src/tokenizer.rs:95-134): plain string
formatting in front of the tokenizer.  The turn markers are the stop strings the scheduler watches for."""
from __future__ import annotations


def gemma4_chat_prompt(user: str) -> str:
    """Single user turn, thinking off, model turn opened (tokenizer.rs:96-98)."""
    return f"<|turn>user\n{user}<turn|>\n<|turn>model\n"


def gemma4_chat_from_messages(messages) -> str:
    """(role, content) pairs with roles system / user / assistant (tokenizer.rs:102-134): system contents are joined
    by blank lines into one leading system turn that starts with `<|think|>`, `assistant` becomes `model`, every other
    role `user`; a model turn is always left open."""
    system, body = [], []
    for role, content in messages:
        if role == "system":
            system.append(content)
            continue
        body.append(f"<|turn>{'model' if role == 'assistant' else 'user'}\n{content}<turn|>\n")
    head = ""
    if system:
        head = "<|turn>system\n<|think|>\n" + "\n\n".join(system) + "<turn|>\n"
    return head + "".join(body) + "<|turn>model\n"
