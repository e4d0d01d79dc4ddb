"""The engine against the plain implementation, under every way of cutting the work,
in 32-bit and in bfloat16, on the tiny configurations."""
import pytest
import torch

import cuttings
import plain_qwen2_moe as plain
from tiny_configs import TINY, prompt

pytestmark = pytest.mark.gpu

# 32-bit: the engine and the oracle differ by summation order only.
TOL_F32 = 1e-4
# bfloat16 against the oracle rounding to bfloat16 at the same places: a value that lands on
# the other side of a rounding boundary moves by one bfloat16 step (2^-8 relative); logits
# here are of order one, so a few such steps stay below 1e-2.
TOL_BF16 = 1e-2
# Routing is a discontinuous choice.  Where the oracle's gap between the last expert chosen and
# the first rejected is within the noise of the precision under test, a correct engine may
# choose the other one, and that position's logits then differ by far more than rounding.  Such
# positions are not compared (later positions see the difference only through one key among
# many and stay within the tolerance).  The gaps are in probability (about 1/experts here);
# the router reads the 32-bit residual, which bfloat16 rounding upstream moves by a few 1e-5 (a
# probability by less), 32-bit summation order by about 1e-8.
MARGIN = {"float32": 1e-6, "bfloat16": 2e-4}

FLOOR = {"float32": 0.95, "bfloat16": 0.9}

LENGTHS = [1, 7, 16, 33, 70, 129]


@pytest.fixture(scope="module")
def oracles(tiny_folders):
    cache = {}

    def get(name, dtype):
        key = (name, dtype)
        if key not in cache:
            cache[key] = plain.PlainModel(tiny_folders[name], compute=torch.float64,
                                          emulate_bf16=(dtype == "bfloat16"))
        return cache[key]
    return get


@pytest.fixture(scope="module")
def engines(tiny_folders):
    from dlm_b200.engine import Engine
    cache = {}

    def get(name, dtype, page_size=16, num_pages=40):
        key = (name, dtype, page_size, num_pages)
        if key not in cache:
            cache[key] = Engine.from_pretrained(tiny_folders[name], dtype=dtype, page_size=page_size,
                                                num_pages=num_pages, max_requests=8, max_context=4096)
        return cache[key]
    return get


_PICKED = {}


def requests_of(name, dtype, oracles, lengths=LENGTHS, base=0):
    """Seeded prompts of the given lengths, each with its per-position routing margins."""
    V = TINY[name]["cfg"]["vocab_size"]
    out = {}
    for i, n in enumerate(lengths):
        key = (name, dtype, base + i, n)
        if key not in _PICKED:
            toks = prompt(base + i, n, V)
            _PICKED[key] = (toks, oracles(name, dtype).router_margins(toks))
        out[f"r{i}"] = _PICKED[key]
    return out


def tokens_of(reqs):
    return {rid: toks for rid, (toks, _) in reqs.items()}


def compare(got, oracle, reqs, dtype):
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    compared = total = 0
    for rid, (toks, margins) in reqs.items():
        ref = oracle.logits(toks)
        total += len(toks)
        for p in range(len(toks)):
            assert (rid, p) in got, f"no logits for {rid} position {p}"
            if float(margins[p]) < MARGIN[dtype]:
                continue
            d = float((got[(rid, p)] - ref[p]).abs().max())
            assert d <= tol, f"request {rid} (length {len(toks)}) position {p}: max abs diff {d:.3e} > {tol}"
            compared += 1
    # the comparison must not be empty: the floors sit just under the smallest share seen
    print(f"compared {compared} of {total} positions ({compared / total:.3f})")
    floor = FLOOR[dtype]
    assert compared >= floor * total, f"only {compared} of {total} positions could be compared"


CASES = [(n, d) for n in TINY for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(name, dtype, engines, oracles):
    reqs = requests_of(name, dtype, oracles)
    got = cuttings.run_trace(engines(name, dtype), cuttings.whole(tokens_of(reqs)))
    compare(got, oracles(name, dtype), reqs, dtype)


@pytest.mark.parametrize("name,dtype", CASES)
def test_tail_decoded_one_by_one(name, dtype, engines, oracles):
    reqs = requests_of(name, dtype, oracles, [33, 70, 129], base=10)
    got = cuttings.run_trace(engines(name, dtype), cuttings.tail_decode(tokens_of(reqs), 32))
    compare(got, oracles(name, dtype), reqs, dtype)


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype, engines, oracles):
    reqs = requests_of(name, dtype, oracles, [16, 70, 129], base=20)
    got = cuttings.run_trace(engines(name, dtype), cuttings.portions(tokens_of(reqs)))
    compare(got, oracles(name, dtype), reqs, dtype)


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("page_size", [16, 64])
def test_mixed_with_few_pages(name, dtype, page_size, engines, oracles):
    reqs = requests_of(name, dtype, oracles, [70, 33, 129, 16, 90, 7, 150, 41], base=30)
    steps, _ = cuttings.mixed(tokens_of(reqs), max_live=4, seed=5)
    peak = cuttings.peak_tokens(steps)
    eng = engines(name, dtype, page_size=page_size, num_pages=peak // page_size)
    got = cuttings.run_trace(eng, steps)
    compare(got, oracles(name, dtype), reqs, dtype)
    for g, st in enumerate(eng.cache.stats()):
        assert st.used_pages == 0 and st.high_water <= peak // page_size
    # the pool was smaller than the sum of the requests: pages were handed out again
    assert sum(-(-len(t) // page_size) for t, _ in reqs.values()) > peak // page_size


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens(name, dtype, engines, oracles):
    V = TINY[name]["cfg"]["vocab_size"]
    reqs = requests_of(name, dtype, oracles, [1, 2, 3, 4], base=50)
    steps = cuttings.tail_decode(tokens_of(reqs), tail=8)       # every token on its own
    got = cuttings.run_trace(engines(name, dtype), steps)
    compare(got, oracles(name, dtype), reqs, dtype)


@pytest.mark.parametrize("name", list(TINY))
def test_cuttings_agree_with_each_other_bf16(name, engines, oracles):
    """Whatever the cut, the same position gives the same logits up to rounding (different
    cuts run different kernels, which sum in different orders)."""
    V = TINY[name]["cfg"]["vocab_size"]
    reqs = {"a": prompt(70, 70, V), "b": prompt(71, 129, V)}
    margins = {rid: oracles(name, "bfloat16").router_margins(t) for rid, t in reqs.items()}
    eng = engines(name, "bfloat16")
    a = cuttings.run_trace(eng, cuttings.whole(reqs))
    b = cuttings.run_trace(eng, cuttings.portions(reqs))
    c = cuttings.run_trace(eng, cuttings.tail_decode(reqs, 32))
    for key in a:
        if float(margins[key[0]][key[1]]) < MARGIN["bfloat16"]:
            continue
        assert float((a[key] - b[key]).abs().max()) <= TOL_BF16
        assert float((a[key] - c[key]).abs().max()) <= TOL_BF16


@pytest.mark.parametrize("name", list(TINY))
def test_long_decoding_fp32(name, engines, oracles):
    """A short prompt and 160 greedy tokens: positions far past the window, many pages."""
    V = TINY[name]["cfg"]["vocab_size"]
    p = prompt(77, 5, V)
    eng = engines(name, "float32")
    out = eng.generate(p, max_new_tokens=160)
    assert len(out) == 160
    # the oracle, fed the engine's own tokens, must choose the same token at every place
    # where its two best logits are further apart than the tolerance
    ref = oracles(name, "float32").logits(p + out[:-1])
    for i, tok in enumerate(out):
        row = ref[len(p) - 1 + i]
        top2 = torch.topk(row, 2).values
        if float(top2[0] - top2[1]) > 10 * TOL_F32:
            assert int(torch.argmax(row)) == tok, f"generated token {i} differs from the oracle's choice"


@pytest.mark.parametrize("name,dtype", CASES)
def test_greedy_generation_through_entry_point(name, dtype, tiny_folders, oracles):
    import dlm_b200
    V = TINY[name]["cfg"]["vocab_size"]
    prompts = [prompt(90 + i, n, V) for i, n in enumerate([1, 7, 16, 33])]
    outs = dlm_b200.generate(tiny_folders[name], prompts, dtype=dtype, max_new_tokens=16, page_size=16,
                             num_pages=32, max_requests=4, max_step_tokens=24)
    oracle = oracles(name, dtype)
    tol = TOL_F32 if dtype == "float32" else TOL_BF16
    for p, out in zip(prompts, outs):
        assert len(out) == 16
        ref = oracle.logits(p + out[:-1])
        for i, tok in enumerate(out):
            row = ref[len(p) - 1 + i]
            top2 = torch.topk(row, 2).values
            if float(top2[0] - top2[1]) > 10 * tol:
                assert int(torch.argmax(row)) == tok


def test_batched_equals_isolated(tiny_folders):
    from dlm_b200.engine import Engine
    V = TINY["B"]["cfg"]["vocab_size"]
    prompts = [prompt(20 + i, n, V) for i, n in enumerate([3, 18, 41, 70, 9, 30])]
    eng = Engine.from_pretrained(tiny_folders["B"], dtype="float32", page_size=16, num_pages=64, max_requests=3,
                                 max_step_tokens=20)
    together = eng.generate(prompts, max_new_tokens=24, temperature=0.8, seed=11)
    alone = [eng.generate(p, max_new_tokens=24, temperature=0.8, seed=11) for p in prompts]
    assert together == alone
    again = eng.generate(prompts, max_new_tokens=24, temperature=0.8, seed=11)
    assert again == together
    other = eng.generate(prompts, max_new_tokens=24, temperature=0.8, seed=12)
    assert other != together


def test_temperature_sampling_matches_oracle_sampler(tiny_folders, oracles):
    """Seeded sampling at temperature 0.8: the engine's tokens are the plain sampler's, fed
    the oracle's logits of the same prefix (checked where the draw is not within rounding of
    a boundary between two candidates)."""
    from dlm_b200.engine import Engine
    V = TINY["B"]["cfg"]["vocab_size"]
    p = prompt(31, 12, V)
    eng = Engine.from_pretrained(tiny_folders["B"], dtype="float32", page_size=16, num_pages=16, max_requests=2)
    out = eng.generate(p, max_new_tokens=24, temperature=0.8, seed=5)
    oracle = oracles("B", "float32")
    rng = plain.SplitMix64(5)
    agree = 0
    for i, tok in enumerate(out):
        row = oracle.logits(p + out[:i])[-1]
        want = plain.sample_topk_topp(row, 0.8, 1.0, 0, 0.0, rng)
        agree += int(want == tok)
    assert agree >= len(out) - 1      # at most one draw may sit on a boundary


def test_preemption_keeps_outputs(tiny_folders):
    """A pool too small for every request at once: some are pre-empted and recomputed, and
    every output is what the request produces alone."""
    from dlm_b200.engine import Engine
    V = TINY["A"]["cfg"]["vocab_size"]
    prompts = [prompt(60 + i, 30, V) for i in range(4)]
    big = Engine.from_pretrained(tiny_folders["A"], dtype="float32", page_size=16, num_pages=64, max_requests=4)
    want = [big.generate(p, max_new_tokens=40) for p in prompts]
    small = Engine.from_pretrained(tiny_folders["A"], dtype="float32", page_size=16, num_pages=10, max_requests=4)
    got = small.generate(prompts, max_new_tokens=40)
    assert got == want
    assert small.stats()["preemptions"] > 0
    assert small.cache.manager.check() == ""
