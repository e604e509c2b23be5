"""The engine at the layer sizes of Mistral 7B (two layers, a vocabulary of 4096), against the
plain implementation, cut three ways.  At these sizes the few-token products split K, so the
decode steps run the path that the measurements time: the norm folded into the products
around it and the q/k/v product that rotates and writes the cache itself
(reference for the order rotate, then cache: src/model/modules/attention.rs:69-75)."""
import numpy as np
import pytest

from helpers_gpu import TinyModel, assert_close
from tiny import REAL_SIZES, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def real(request):
    return TinyModel("real", request.param, seed=5, max_tokens=2048, cfg=REAL_SIZES)


def _requests(m, lengths, seed):
    rng = np.random.default_rng(seed)
    return [random_tokens(rng, n, m.cfg["vocab_size"]) for n in lengths]


def test_whole(real):
    """One prompt of 300 tokens (the many-token product kernel and the tensor-core prefill
    attention) and a short one."""
    for toks in _requests(real, [300, 9], 1):
        (s,) = real.engine.start_sequences(1)
        got = real.step_np([s], [toks], "all")
        real.engine.end_sequences([s])
        assert_close(got, real.reference(toks), real.dtype, f"whole n={len(toks)}")


def test_last_32_one_by_one_runs_the_folded_path(real):
    from torchless_rs_b200.csrc import ops
    (toks,) = _requests(real, [140], 2)
    n = len(toks)
    (s,) = real.engine.start_sequences(1)
    got = [real.step_np([s], [toks[:n - 32]], "all")]
    before = ops.launch_counts()
    for t in toks[n - 32:]:
        got.append(real.step_np([s], [[t]], "last"))
    during = ops.counts_since(before)
    real.engine.end_sequences([s])
    assert_close(np.concatenate(got), real.reference(toks), real.dtype, "last 32")
    if real.dtype == "bfloat16":
        layers = real.cfg["num_hidden_layers"]
        # per step: the first layer's first norm and the final norm run as kernels, every other
        # norm is folded; no rotation kernel; five products per layer minus nothing, plus the head
        assert during.get("rope_cache_write", 0) == 0, during
        assert during.get("rmsnorm", 0) == 32 * 2, during
        assert during.get("gemm_tc", 0) == 32 * (4 * layers + 1), during
        assert during.get("gemm_generic", 0) == 0 and during.get("attn_generic", 0) == 0, during


@pytest.mark.parametrize("batch", [3, 16])
def test_unequal_batch_then_decode(real, batch):
    """Prompts of unequal lengths start together; then every request goes on one token per
    step until its tokens run out (batches of 3 and of 16: K is split 8 and fewer ways)."""
    rng = np.random.default_rng(3 + batch)
    lens = [int(x) for x in rng.integers(8, 90, size=batch)]
    lens[0], lens[-1] = 70, 12
    reqs = _requests(real, lens, 4 + batch)
    ahead = [int(x) for x in rng.integers(2, 8, size=batch)]   # tokens left for decoding
    slots = real.engine.start_sequences(batch)
    pre = [len(r) - a for r, a in zip(reqs, ahead)]
    out = real.step_np(slots, [r[:p] for r, p in zip(reqs, pre)], "all")
    got, o = [[] for _ in reqs], 0
    for i, p in enumerate(pre):
        got[i].append(out[o:o + p]); o += p
    fed, live = list(pre), list(range(batch))
    while live:
        out = real.step_np([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1]); fed[i] += 1
        done = [i for i in live if fed[i] >= len(reqs[i])]
        real.engine.end_sequences([slots[i] for i in done])
        live = [i for i in live if i not in done]
    real.engine.cache.check()
    for i, r in enumerate(reqs):
        assert_close(np.concatenate(got[i]), real.reference(r), real.dtype, f"request {i} (n={len(r)})")
    real.engine.check_kernels()
