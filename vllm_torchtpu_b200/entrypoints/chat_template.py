"""Chat messages -> prompt token ids.

With a Hugging Face tokenizer its own template is used.  ``continue_final_message`` asks the model to go on
writing the last (assistant) message instead of opening a new turn: tokenizers whose template supports the
flag get it; for the others (templates that always close the final message, as the DeepSeek-V4 one does) the
prompt is rendered with the final message removed and a generation prompt added, and the text of that
message is appended after it, which yields the same tokens as an open assistant turn.  Without a tokenizer
template a plain ``role: content`` transcript is used.
(reference: src/vllm_torchtpu/tokenizers.py:30-81)"""
from __future__ import annotations


def build_chat_prompt(tokenizer, encode, messages: list, add_generation_prompt: bool = True,
                      continue_final_message: bool = False, chat_template_kwargs: dict | None = None) -> list:
    if continue_final_message:
        if not messages or messages[-1].get("role") != "assistant":
            raise ValueError("continue_final_message needs a final assistant message")
        if add_generation_prompt:
            add_generation_prompt = False        # the two are exclusive; continuing wins as in the chat API
    kwargs = dict(chat_template_kwargs or {})
    if tokenizer is not None and hasattr(tokenizer, "apply_chat_template"):
        if not continue_final_message:
            return list(tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                      tokenize=True, **kwargs))
        try:
            return list(tokenizer.apply_chat_template(messages, add_generation_prompt=False, tokenize=True,
                                                      continue_final_message=True, **kwargs))
        except (TypeError, ValueError):
            # a template without the flag: open a fresh assistant turn and put the partial answer inside it
            head = tokenizer.apply_chat_template(messages[:-1], add_generation_prompt=True, tokenize=False, **kwargs)
            return list(encode(head + str(messages[-1].get("content", ""))))
    lines = [f"{m.get('role', 'user')}: {m.get('content', '')}" for m in messages]
    text = "\n".join(lines)
    if continue_final_message:
        return list(encode(text))
    return list(encode(text + ("\nassistant:" if add_generation_prompt else "")))
