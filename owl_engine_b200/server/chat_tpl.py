"""Chat template rendering (HF ``chat_template.jinja`` semantics) with jinja2.

``ChatTemplate.render(messages, tools=..., add_generation_prompt=True, **kwargs)`` produces the
prompt text. A model directory's own template is used when present; otherwise the built-in
ChatML-style template (system / user / assistant / tool roles, ``<tool_call>`` blocks, optional
thinking) is used. ``chat_template_kwargs`` of a request are passed through as template variables;
a template-vars file supplies defaults. Reference counterpart: ``apps/server/src/chat_tpl.rs``.
"""
from __future__ import annotations

import json
from pathlib import Path

import jinja2

BUILTIN = r"""
{%- if tools %}
<|im_start|>system
{%- if messages and messages[0].role == 'system' %}
{{ messages[0].content }}
{%- endif %}

# Tools

You may call one or more functions. Function signatures are inside <tools></tools>:
<tools>
{%- for tool in tools %}
{{ tool | tojson }}
{%- endfor %}
</tools>

For each call return a JSON object inside <tool_call></tool_call>:
<tool_call>
{"name": <function-name>, "arguments": <args-json-object>}
</tool_call><|im_end|>
{%- elif messages and messages[0].role == 'system' %}
<|im_start|>system
{{ messages[0].content }}<|im_end|>
{%- endif %}
{%- for m in messages %}
{%- if m.role == 'system' and loop.first %}
{%- elif m.role == 'assistant' %}
<|im_start|>assistant
{%- if m.reasoning_content %}
<think>
{{ m.reasoning_content }}
</think>
{%- endif %}
{{ m.content or '' }}
{%- for tc in m.tool_calls or [] %}
<tool_call>
{"name": "{{ tc.function.name }}", "arguments": {{ tc.function.arguments if tc.function.arguments is string else tc.function.arguments | tojson }}}
</tool_call>
{%- endfor %}<|im_end|>
{%- elif m.role == 'tool' %}
<|im_start|>user
<tool_response>
{{ m.content }}
</tool_response><|im_end|>
{%- else %}
<|im_start|>{{ m.role }}
{{ m.content }}<|im_end|>
{%- endif %}
{%- endfor %}
{%- if add_generation_prompt %}
{{ '<|im_start|>assistant\n' }}
{%- if enable_thinking is defined and enable_thinking is false %}
{{- '<think>\n\n</think>\n\n' }}
{%- endif %}
{%- endif -%}
"""


def _flatten_content(content) -> str:
    """OpenAI content parts -> text with image placeholders."""
    if isinstance(content, str) or content is None:
        return content or ""
    out = []
    for part in content:
        if part.get("type") == "text":
            out.append(part.get("text", ""))
        elif part.get("type") in ("image_url", "image"):
            out.append("<|vision_start|><|image_pad|><|vision_end|>")
    return "".join(out)


class ChatTemplate:
    def __init__(self, template_path: str = "", vars_path: str = ""):
        env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False, keep_trailing_newline=True)
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False)
        env.globals["raise_exception"] = self._raise
        src = Path(template_path).read_text() if template_path else BUILTIN
        self.template = env.from_string(src)
        self.defaults = json.loads(Path(vars_path).read_text()) if vars_path else {}

    @staticmethod
    def _raise(msg):
        raise jinja2.TemplateError(msg)

    def render(self, messages: list, tools: list | None = None, add_generation_prompt: bool = True, **kwargs) -> str:
        msgs = [dict(m, content=_flatten_content(m.get("content"))) for m in messages]
        ctx = dict(self.defaults)
        ctx.update(kwargs)
        text = self.template.render(messages=msgs, tools=tools or None, add_generation_prompt=add_generation_prompt, **ctx)
        return text.lstrip("\n")
