"""Streaming invariants of the output splitter: what a turn's text is divided into must not depend on how the token
stream happened to cut it, and no character may be lost or invented."""
import json

from hypothesis import given, settings, strategies as st

from owl_engine_b200.server.toolcall import ChannelSplitter

TOOLS = [{"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {
    "city": {"type": "string"}, "days": {"type": "integer"}}}}}]

PIECES = [
    "plain words ", "and more, with < and > and <b>tags</b> ", "\n", "<think>", "</think>", "reasoning about it ",
    "<tool_call>", "</tool_call>", '{"name": "get_weather", "arguments": {"city": "Oslo", "days": 2}}',
    "<function=get_weather>", "<parameter=city>", "Oslo", "</parameter>", "</function>", "<tool", "</thi", "<|im_end|>",
    "<thinking>", "</thinking>", "{", "}", '"', "é", "日本",
    "<thought>", "</thought>", "<function_calls>", "</function_calls>", '<invoke name="get_weather">', "</invoke>",
    '<parameter name="city">', "  ", "\n\n", "<function=", "<function=unknown_tool>", '{"name": "get_weather"', "</",
]


def run(chunks, start_in_think=False):
    sp = ChannelSplitter(start_in_think=start_in_think, tools=TOOLS)
    ev = []
    for c in chunks:
        ev += sp.feed(c)
    ev += sp.finish()
    # merge adjacent text / reasoning events: their boundaries are an artefact of the chunking
    merged = []
    for e in ev:
        if merged and e[0] in ("text", "reasoning") and merged[-1][0] == e[0]:
            merged[-1] = (e[0], merged[-1][1] + e[1])
        else:
            merged.append(tuple(e))
    return merged, sp


def cuts(text, points):
    pts = sorted({p % (len(text) + 1) for p in points})
    out, last = [], 0
    for p in pts:
        out.append(text[last:p])
        last = p
    out.append(text[last:])
    return [c for c in out if c]


@settings(max_examples=300, deadline=None)
@given(st.lists(st.sampled_from(PIECES), min_size=1, max_size=14), st.lists(st.integers(0, 10 ** 6), max_size=12), st.booleans())
def test_events_do_not_depend_on_the_chunking(pieces, points, in_think):
    text = "".join(pieces)
    whole, _ = run([text], in_think)
    chunked, _ = run(cuts(text, points), in_think)
    by_char, _ = run(list(text), in_think)
    assert chunked == whole and by_char == whole


@settings(max_examples=200, deadline=None)
@given(st.text(alphabet=st.characters(blacklist_characters="<", blacklist_categories=("Cs",)), max_size=200),
       st.lists(st.integers(0, 10 ** 6), max_size=8))
def test_text_without_markers_passes_through_unchanged(text, points):
    ev, sp = run(cuts(text, points) or [""])
    assert "".join(e[1] for e in ev if e[0] == "text") == text and all(e[0] == "text" for e in ev)
    assert sp.n_calls == 0 and sp.malformed == 0


@settings(max_examples=150, deadline=None)
@given(st.text(alphabet="abc xyz.\n", max_size=40), st.text(alphabet="abc xyz.\n", max_size=40),
       st.sampled_from(["Oslo", "New York", 'a "quoted" city', "日本"]), st.integers(0, 9), st.lists(st.integers(0, 10 ** 6), max_size=10))
def test_a_well_formed_call_is_found_whatever_surrounds_it(before, after, city, days, points):
    call = json.dumps({"name": "get_weather", "arguments": {"city": city, "days": days}}, ensure_ascii=False)
    text = f"{before}<tool_call>\n{call}\n</tool_call>{after}"
    ev, sp = run(cuts(text, points))
    calls = [e for e in ev if e[0] == "tool_call"]
    assert len(calls) == 1 and sp.malformed == 0
    name, args = calls[0][1]["name"], calls[0][1]["arguments"]
    assert name == "get_weather" and json.loads(args) == {"city": city, "days": days}
    shown = "".join(e[1] for e in ev if e[0] == "text")
    assert shown.replace("\n", "").replace(" ", "") == (before + after).replace("\n", "").replace(" ", "")


@settings(max_examples=300, deadline=None)
@given(st.text(alphabet="ab <>\nSTOPé日", max_size=60), st.lists(st.sampled_from(["STOP", "\n\n", "ab", "é日", "<b>"]), min_size=1, max_size=3,
                                                                   unique=True))
def test_streamed_content_ends_before_the_first_stop_string_whatever_the_token_boundaries(text, stops):
    """Through the whole response path (byte tokens -> incremental detokeniser -> splitter -> stop holding): the streamed
    content is the text up to the first stop string, the chunks never contain a piece of a stop string that then completes,
    and multi-byte characters are never cut."""
    from owl_engine_b200.engine.tokenizer import ByteTokenizer, StreamDecoder
    from owl_engine_b200.server.openai import Streamer

    tok = ByteTokenizer()
    s = Streamer("m", StreamDecoder(tok), stops)
    chunks = []
    for t in tok.encode(text):
        chunks += s.on_token(t)
        if s.stopped:
            break
    chunks += s.finish("length", {"prompt_tokens": 1, "completion_tokens": 1}, False)
    got = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    cut = min((text.find(x) for x in stops if x in text), default=len(text))
    want = text[:cut]
    # the splitter drops nothing here except marker look-alikes it must hold until they are decided; "<b>" is plain text
    assert got == want, (got, want)
    assert chunks[-1]["choices"][0]["finish_reason"] == ("stop" if cut < len(text) else "length")
    for c in chunks:
        piece = c["choices"][0]["delta"].get("content", "")
        assert "\\ufffd" not in piece.encode("unicode_escape").decode()


@settings(max_examples=300, deadline=None)
@given(st.text(alphabet=st.characters(blacklist_categories=("Cs",)), max_size=80),
       st.lists(st.sampled_from(["<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "<|image_pad|>"]), max_size=4),
       st.randoms(use_true_random=False))
def test_byte_tokenizer_round_trips_and_the_stream_decoder_never_cuts_a_character(text, specials, rnd):
    from owl_engine_b200.engine.tokenizer import ByteTokenizer, StreamDecoder

    tok = ByteTokenizer()
    parts = [text[i:i + 7] for i in range(0, len(text), 7)] or [""]
    for sp in specials:
        parts.insert(rnd.randrange(len(parts) + 1), sp)
    full = "".join(parts)
    ids = tok.encode(full)
    assert tok.decode(ids) == full
    assert all(0 <= t < tok.vocab_size for t in ids)
    dec, out = StreamDecoder(tok), []
    for t in ids:
        piece = dec.push(t)
        assert "\\ufffd" not in piece.encode("unicode_escape").decode() or "\\ufffd" in full.encode("unicode_escape").decode()
        out.append(piece)
    assert "".join(out) == full
