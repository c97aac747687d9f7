import json

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
    full = 'Hi<think>plan a\nb</think>\nAnswer <tool_call>\n{"name": "f", "arguments": {"x": 1}}\n</tool_call>\ntail'
    for size in (1, 2, 3, 7, 1000):
        ev = run([full[i:i + size] for i in range(0, len(full), size)])
        assert join(ev, "reasoning") == "plan a\nb"
        assert join(ev, "text") == "Hi\nAnswer \ntail"
        calls = [e[1] for e in ev if e[0] == "tool_call"]
        assert len(calls) == 1 and calls[0]["name"] == "f" and json.loads(calls[0]["arguments"]) == {"x": 1}


def test_splitter_xml_form_and_lookalikes_and_unterminated():
    ev = run(["<tool_call><function=get_w><parameter=city>Paris</parameter><parameter=n>3</parameter></function></tool_call>"])
    assert json.loads(ev[0][1]["arguments"]) == {"city": "Paris", "n": 3}
    ev = run(["a < b <thin", "g> and <tool_", "x>"])
    assert join(ev, "text") == "a < b <thing> and <tool_x>"
    ev = run(["<tool_call>not json"])
    assert join(ev, "text") == "<tool_call>not json"
    ev = run(["reasoning here</think>ok"], start_in_think=True)
    assert join(ev, "reasoning") == "reasoning here" and join(ev, "text") == "ok"
    assert parse_tool_body("garbage") is None


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
