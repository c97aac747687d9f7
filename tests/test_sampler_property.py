"""Properties of the host sampler: the draw is a function of (seed, turn, step), stays inside the candidates and their top-k /
top-p cut, and the extreme settings reduce to the arg max."""
import math

from hypothesis import given, settings, strategies as st

from owl_engine_b200.engine import sampler as S

cands = st.lists(st.tuples(st.integers(0, 10 ** 5), st.floats(-30, 30, allow_nan=False)), min_size=1, max_size=32,
                 unique_by=lambda c: c[0])
params = st.builds(S.SamplingParams, st.just("sampling"), st.floats(0.0, 3.0), st.integers(1, 40), st.floats(0.01, 1.0),
                   st.floats(0.8, 1.5), st.integers(0, 2 ** 40))


@settings(max_examples=400)
@given(cands, params, st.integers(0, 1000), st.integers(0, 5000), st.sets(st.integers(0, 10 ** 5), max_size=6))
def test_draws_are_reproducible_and_stay_inside_the_cut(c, p, turn, step, history):
    tok = S.sample(c, p, turn, step, history)
    assert tok == S.sample(list(reversed(c)), p, turn, step, history)        # a function of the values, not of their order
    assert tok in {t for t, _ in c}
    pen = S.apply_rep_penalty(c, history, p.rep_penalty)
    dist = S.distribution(pen, p)
    assert abs(sum(q for _, q in dist) - 1.0) < 1e-9 and len(dist) <= min(p.topk, len(c))
    assert all(a[1] >= b[1] - 1e-12 for a, b in zip(dist, dist[1:]))          # sorted by probability
    if p.temp > 0:
        assert tok in {t for t, _ in dist}
    top = sorted(pen, key=lambda x: (-x[1], x[0]))[:p.topk]
    assert {t for t, _ in dist} <= {t for t, _ in top}


@settings(max_examples=200)
@given(cands, st.integers(0, 2 ** 40), st.integers(0, 100), st.integers(0, 100))
def test_extreme_settings_reduce_to_the_arg_max(c, seed, turn, step):
    best = max(c, key=lambda x: x[1])[1]
    winners = {t for t, l in c if l == best}
    assert S.sample(c, S.SamplingParams("greedy"), turn, step) in winners
    assert S.sample(c, S.SamplingParams("sampling", 0.0, 20, 0.95, 1.0, seed), turn, step) in winners
    assert S.sample(c, S.SamplingParams("sampling", 1.0, 1, 1.0, 1.0, seed), turn, step) in winners          # top-k = 1
    if len(winners) == 1 and all(l <= best - 1e-3 for t, l in c if t not in winners):
        assert S.sample(c, S.SamplingParams("sampling", 1e-4, 20, 1.0, 1.0, seed), turn, step) in winners    # temperature -> 0


@settings(max_examples=60)
@given(st.integers(0, 2 ** 60))
def test_the_generator_is_uniform_enough_and_never_stalls(seed):
    r = S.XorShift64Star(seed)
    xs = [r.uniform() for _ in range(2000)]
    assert all(0.0 <= x < 1.0 for x in xs) and 0.45 < sum(xs) / len(xs) < 0.55 and len(set(xs)) > 1990
    assert S.step_seed(seed, 1, 2) != S.step_seed(seed, 2, 1) and S.step_seed(seed, 0, 0) != 0
    assert not math.isnan(xs[0])


@settings(max_examples=300)
@given(st.lists(st.one_of(st.tuples(st.just("append"), st.lists(st.integers(0, 6), min_size=1, max_size=9)),
                          st.tuples(st.just("truncate"), st.integers(0, 30)),
                          st.tuples(st.just("rewrite"), st.lists(st.integers(0, 6), min_size=0, max_size=30))), min_size=1, max_size=25),
       st.integers(1, 3), st.integers(3, 8), st.integers(1, 5))
def test_lookup_history_buffer_always_answers_like_a_fresh_search(ops, nmin, nmax, k):
    """The lookup keeps a growing array per sequence instead of converting the token list every round: whatever happens to
    the list (appends, rollbacks, announced rewrites), its answer equals a search over the list itself;
    and the answer is a real continuation of a real earlier occurrence."""
    from types import SimpleNamespace

    from owl_engine_b200.engine.spec import LookupDraft, suffix_lookup

    seq = SimpleNamespace(tokens=[], tokens_epoch=0)
    eng = SimpleNamespace(seqs={7: seq})
    lk = LookupDraft(nmin, nmax)
    for op, arg in ops:
        if op == "append":
            seq.tokens += arg
        elif op == "truncate":
            del seq.tokens[max(0, len(seq.tokens) - arg):]
        else:
            seq.tokens[:] = arg
            seq.tokens_epoch += 1                                          # in-place edits are announced
        got = lk.find(eng, 7, k)
        want = suffix_lookup(list(seq.tokens), k, nmin, nmax)
        assert got == want
        if got is not None:
            follow, m = got
            t = seq.tokens
            assert nmin <= m <= nmax and 1 <= len(follow) <= k
            ends = [e for e in range(m - 1, len(t) - 1) if t[e - m + 1:e + 1] == t[len(t) - m:] and t[e + 1:e + 1 + len(follow)] == follow]
            assert ends                                                    # it followed an earlier occurrence of the last m tokens


@settings(max_examples=300)
@given(st.lists(st.one_of(st.integers(0, 265), st.sampled_from(list("aé€😀 \n".encode()))), min_size=0, max_size=60))
def test_streamed_text_is_the_decoded_text_and_each_token_decodes_a_short_window(ids):
    """Whatever the ids (valid UTF-8, stray continuation bytes, specials), the pieces a stream emits join to the decoded
    whole, except for a tail that still ends in an incomplete character; and no push decodes more than the two latest
    emissions' worth of ids."""
    from owl_engine_b200.engine.tokenizer import ByteTokenizer, StreamDecoder

    class Counting(ByteTokenizer):
        longest = 0

        def decode(self, ids):
            ids = list(ids)
            self.longest = max(self.longest, len(ids))
            return super().decode(ids)

    tok = Counting()
    d = StreamDecoder(tok)
    out = "".join(d.push(t) for t in ids)
    whole = ByteTokenizer().decode(ids)
    assert whole.startswith(out)
    rest = whole[len(out):]
    assert rest == "" or rest.endswith("�")
    text = [ord("x")] * 500
    tok2 = Counting()
    d2 = StreamDecoder(tok2)
    assert "".join(d2.push(t) for t in text) == "x" * 500 and tok2.longest <= 2


@settings(max_examples=300)
@given(st.lists(st.one_of(st.sampled_from(["<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "<|image_pad|>", "<", "|", ">", "im_"]),
                          st.text(max_size=6)), max_size=12))
def test_byte_tokenizer_round_trips_text_with_specials_and_their_fragments(parts):
    """encode then decode gives the text back (lone surrogates aside, which UTF-8 cannot carry), specials take one id each,
    and fragments of specials stay bytes."""
    from owl_engine_b200.engine.tokenizer import ByteTokenizer

    tok = ByteTokenizer()
    text = "".join(parts)
    try:
        text.encode("utf-8")
    except UnicodeEncodeError:
        return
    ids = tok.encode(text)
    assert tok.decode(ids) == text
    assert sum(1 for t in ids if t >= 256) == sum(text.count(s) for s in tok.SPECIALS)
    assert all(0 <= t < 256 + len(tok.SPECIALS) for t in ids)
