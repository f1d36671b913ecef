"""Chat templates: render a message list to a prompt string.

The reference carries its own minimal Jinja interpreter (JinjaEngine / JinjaExpr,
src/HartsyInference.LLM/ChatTemplates/) plus ChatML and raw fallbacks; here ``jinja2`` renders the
template stored in the checkpoint (``tokenizer_config.json`` ``chat_template`` or the GGUF key
``tokenizer.chat_template``) inside a sandbox, with the same fallbacks.
"""
from __future__ import annotations

from typing import Optional, Sequence

CHATML = ("{% for message in messages %}{{ '<|im_start|>' + message['role'] + '\n' + message['content'] + "
          "'<|im_end|>' + '\n' }}{% endfor %}{% if add_generation_prompt %}{{ '<|im_start|>assistant\n' }}{% endif %}")
RAW = "{% for message in messages %}{{ message['content'] }}{% if not loop.last %}\n{% endif %}{% endfor %}"
LLAMA3 = ("{{ bos_token }}{% for message in messages %}{{ '<|start_header_id|>' + message['role'] + "
          "'<|end_header_id|>\n\n' + message['content'] | trim + '<|eot_id|>' }}{% endfor %}"
          "{% if add_generation_prompt %}{{ '<|start_header_id|>assistant<|end_header_id|>\n\n' }}{% endif %}")

REGISTRY = {"chatml": CHATML, "raw": RAW, "llama3": LLAMA3}


def _raise(msg: str):
    raise ValueError(msg)


class ChatTemplate:
    def __init__(self, source: Optional[str] = None, bos_token: str = "", eos_token: str = ""):
        from jinja2.sandbox import ImmutableSandboxedEnvironment
        self.source = REGISTRY.get(source or "chatml", source or CHATML)
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = _raise
        import datetime
        env.globals["strftime_now"] = lambda fmt: datetime.datetime.now().strftime(fmt)
        self._tpl = env.from_string(self.source)
        self.bos_token, self.eos_token = bos_token, eos_token

    def render(self, messages: Sequence[dict], add_generation_prompt: bool = True, tools: Optional[list] = None,
               enable_thinking: Optional[bool] = None, **extra) -> str:
        kw = dict(messages=list(messages), add_generation_prompt=add_generation_prompt, bos_token=self.bos_token,
                  eos_token=self.eos_token, tools=tools, **extra)
        if enable_thinking is not None:
            kw["enable_thinking"] = enable_thinking
        return self._tpl.render(**kw)

    @staticmethod
    def for_arch(arch: str) -> "ChatTemplate":
        if arch.startswith("llama"):
            return ChatTemplate("llama3", bos_token="<|begin_of_text|>")
        return ChatTemplate("chatml")
