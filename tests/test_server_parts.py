"""Server parts without a server: the output splitter on recorded shapes, the repeat guard, the chat template, exact rejection sampling."""
import json

import pytest

from owl_engine_b200.server.chat_tpl import ChatTemplate
from owl_engine_b200.server.toolcall import ChannelSplitter, RepeatGuard, parse_tool_body


def run(chunks, **kw):
    sp = ChannelSplitter(**kw)
    ev = []
    for c in chunks:
        ev += sp.feed(c)
    return ev + sp.finish()


def join(ev, ch):
    return "".join(e[1] for e in ev if e[0] == ch)


def test_splitter_channels_and_partial_tags():
    full = 'Hi<think>plan a\nb</think>\n\nAnswer <tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call>\ntail'
    for size in (1, 2, 3, 7, 1000):
        ev = run([full[i:i + size] for i in range(0, len(full), size)])
        assert join(ev, "reasoning") == "plan a\nb"
        assert join(ev, "text") == "HiAnswer \ntail"        # the template's two line feeds after the closing marker are not content
        calls = [e[1] for e in ev if e[0] == "tool_call"]
        assert len(calls) == 1 and calls[0]["name"] == "f" and json.loads(calls[0]["arguments"]) == {"x": 1}


def test_splitter_xml_form_and_lookalikes_and_unterminated():
    ev = run(["<tool_call><function=get_w><parameter=city>Paris</parameter><parameter=n>3</parameter></function></tool_call>"])
    assert json.loads(ev[0][1]["arguments"]) == {"city": "Paris", "n": 3}
    ev = run(["a < b <thin", "g> and <tool_", "x>"])
    assert join(ev, "text") == "a < b <thing> and <tool_x>"
    ev = run(["<tool_call>not json"])
    assert [e[0] for e in ev] == ["malformed"] and ev[0][1]["kind"] == "unclosed" and join(ev, "text") == ""
    ev = run(["reasoning here</think>ok"], start_in_think=True)
    assert join(ev, "reasoning") == "reasoning here" and join(ev, "text") == "ok"
    import pytest
    from owl_engine_b200.server.toolcall import Malformed

    with pytest.raises(Malformed):
        parse_tool_body("garbage")


TOOLS = [{"type": "function", "function": {"name": "bash", "parameters": {"properties": {
    "timeout": {"type": "integer"}, "cmd": {"type": "string"}, "v": {"anyOf": [{"type": "null"}, {"type": "boolean"}]},
    "xs": {"type": "array"}}}}}]


def test_splitter_emits_at_function_close_and_types_by_schema():
    x = ('<tool_call>\n<function=bash>\n<parameter=cmd>\n123\n</parameter>\n<parameter=timeout>"30.0"</parameter>'
         '<parameter=v>True</parameter><parameter=xs>[1, 2]</parameter></function>')
    sp = ChannelSplitter(tools=TOOLS)
    ev = []
    for c in x:
        ev += sp.feed(c)
    # complete at </function>: the call is out before the wrapper closes
    assert [e[0] for e in ev] == ["tool_call"]
    assert json.loads(ev[0][1]["arguments"]) == {"cmd": "123", "timeout": 30, "v": True, "xs": [1, 2]}   # cmd stays a string
    ev = []
    for c in " \n <function=bash><parameter=cmd>ls</parameter></function>\n</tool_call>after":
        ev += sp.feed(c)
    ev += sp.finish()
    assert [e[0] for e in ev if e[0] == "tool_call"] == ["tool_call"] and ev[0][1]["index"] == 1
    assert join(ev, "text") == "after"                     # white space between the blocks belongs to the template
    assert sp.n_calls == 2 and sp.malformed == 0 and any(t.startswith("tool #1 bash") for t in sp.trace())


def test_splitter_aliases_bare_invoke_and_strays():
    from owl_engine_b200.server.toolcall import NS_PREFIX as NS

    y = ('<thinking>a</thinking>\n\nB<function_calls>\n<invoke name="bash">\n<parameter name="cmd">ls -l</parameter>\n'
         '</invoke>\n<invoke name="g"></invoke></function_calls>C</think>D<thought>e</thought>')
    for size in (1, 5, 1000):
        sp = ChannelSplitter(tools=TOOLS)
        ev = []
        for i in range(0, len(y), size):
            ev += sp.feed(y[i:i + size])
        ev += sp.finish()
        assert join(ev, "reasoning") == "ae" and join(ev, "text") == "BCD"
        calls = [e[1] for e in ev if e[0] == "tool_call"]
        assert [(c["name"], json.loads(c["arguments"])) for c in calls] == [("bash", {"cmd": "ls -l"}), ("g", {})]
        assert sp.strays == 1                               # the closing reasoning marker in text state is swallowed, counted
    # bare function block, inside the reasoning block, no wrapper at all
    ev = run(["thinking <function=bash><parameter=cmd>pwd</parameter></function> done"], start_in_think=True)
    assert [e[1]["name"] for e in ev if e[0] == "tool_call"] == ["bash"] and join(ev, "reasoning") == "thinking "
    # a namespace prefix on the invoke tags, a Qwen body inside the invoke wrapper, a JSON body inside it
    ev = run([f'<function_calls><{NS}invoke name="bash"><{NS}parameter name="cmd">x</{NS}parameter></{NS}invoke></function_calls>'])
    assert json.loads(ev[0][1]["arguments"]) == {"cmd": "x"}
    ev = run(['<function_calls><function=bash><parameter=cmd>y</parameter></function></function_calls>'])
    assert ev[0][0] == "tool_call" and json.loads(ev[0][1]["arguments"]) == {"cmd": "y"}
    ev = run(['<function_calls>{"name": "bash", "arguments": {"cmd": "z"}}</function_calls>'])
    assert ev[0][0] == "tool_call" and json.loads(ev[0][1]["arguments"]) == {"cmd": "z"}


def test_splitter_lenient_json_salvage_and_malformed():
    from owl_engine_b200.server.toolcall import lenient_json

    ev = run(["<tool_call>{'name': 'f', arguments: {a: 1, b: [1,2,], c: True}, } trailing words</tool_call>"])
    assert ev[0][0] == "tool_call" and json.loads(ev[0][1]["arguments"]) == {"a": 1, "b": [1, 2], "c": True}
    v, repaired = lenient_json('{"name": "f", "arguments": {"a": .5, "b": 1., // note\n "d": None')
    assert repaired and v == {"name": "f", "arguments": {"a": 0.5, "b": 1.0, "d": None}}
    # cut off before the closing marker, body whole: salvaged; body not whole: malformed, never text
    ev = run(['<tool_call>{"name": "f", "arguments": {"a": 1}}'])
    assert ev[0][0] == "tool_call"
    ev = run(['<tool_call>{"name": "f", "arguments": {"a": '])
    assert [e[0] for e in ev] == ["malformed"]
    ev = run(["<tool_call><function=bash><parameter=cmd>ls"])
    assert [e[0] for e in ev] == ["malformed"] and ev[0][1]["kind"] == "unclosed"
    ev = run(['<tool_call>{"arguments": {"a": 1}}</tool_call>ok'])
    assert ev[0][0] == "malformed" and ev[0][1]["kind"] == "json_no_name" and join(ev, "text") == "ok"
    # arguments given as a string stay a valid JSON string
    ev = run(['<tool_call>{"name": "f", "arguments": "{\\"a\\": 2}"}</tool_call>'])
    assert json.loads(ev[0][1]["arguments"]) == {"a": 2}
    # tool parsing off: the markers are text
    ev = run(["a<tool_call>b</tool_call>"], parse_tools=False)
    assert join(ev, "text") == "a<tool_call>b</tool_call>"


def test_repeat_guard():
    g = RepeatGuard(3)
    c = {"name": "f", "arguments": "{}"}
    assert [g.observe("s", c) for _ in range(3)] == [False, False, True]
    assert g.observe("s", {"name": "g", "arguments": "{}"}) is False


def test_builtin_template_renders_tools_and_roles():
    t = ChatTemplate()
    msgs = [{"role": "system", "content": "sys"}, {"role": "user", "content": [{"type": "text", "text": "look "},
            {"type": "image_url", "image_url": {"url": "data:..."}}]},
            {"role": "assistant", "content": "", "tool_calls": [{"function": {"name": "f", "arguments": '{"a": 1}'}}]},
            {"role": "tool", "content": "42"}]
    out = t.render(msgs, tools=[{"type": "function", "function": {"name": "f"}}], enable_thinking=False)
    assert out.startswith("<|im_start|>system") and "<tools>" in out and "<|image_pad|>" in out
    assert '<tool_call>\n{"name": "f", "arguments": {"a": 1}}' in out and "<tool_response>\n42" in out
    assert out.rstrip().endswith("</think>")
    plain = t.render([{"role": "user", "content": "hi"}])
    assert plain == "<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"


def test_rejection_sampling_is_exact():
    """accept_rejection draws from the target distribution whatever the proposal is."""
    import random
    from collections import Counter

    from owl_engine_b200.engine.spec import accept_greedy, accept_rejection

    assert accept_greedy([5, 6, 7], [5, 6, 9, 1]) == 2 and accept_greedy([], [3]) == 0
    p0, p1 = {1: 0.5, 2: 0.3, 3: 0.2}, {4: 0.9, 5: 0.1}
    q0 = {1: 0.1, 2: 0.8, 3: 0.1}
    rng = random.Random(0)
    first, n = Counter(), 20000
    for _ in range(n):
        d = rng.choices(list(q0), weights=list(q0.values()))[0]      # the draft is sampled from q
        m, nxt = accept_rejection([d], [q0], [p0, p1], rng)
        first[d if m == 1 else nxt] += 1
    for t, pv in p0.items():
        assert abs(first[t] / n - pv) < 0.015


def test_runaway_nesting_in_a_tool_block_is_a_malformed_item_not_a_crash():
    from owl_engine_b200.server.toolcall import ChannelSplitter, lenient_json

    for s in ("[" * 100000, '{"a":' * 50000):
        with pytest.raises(ValueError):
            lenient_json(s)
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"a": {"type": "array"}}}}}]
    deep = "[" * 50000 + "]" * 50000
    sp = ChannelSplitter(tools=tools)
    ev = sp.feed('<tool_call>{"name": "f", "arguments": ' + deep + "}</tool_call>") + sp.finish()
    assert [e[0] for e in ev] == ["malformed"] and sp.malformed == 1
    sp = ChannelSplitter(tools=tools)
    ev = sp.feed("<tool_call><function=f><parameter=a>" + deep + "</parameter></function></tool_call>after") + sp.finish()
    assert [e[0] for e in ev] == ["tool_call", "text"]              # the argument stays a string; the stream goes on
