"""Each kernel alone against a plain 32-bit reference written here, at sizes other
than the engine tests use."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
PAGE = 64


def _ops(dtype):
    from torchless_rs_b200.csrc import ops
    return ops.core_ops(dtype)


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


# ---------------------------------------------------------------------------
# embedding, norm, SiLU-gate
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    o = _ops(dtype)
    table = _rand((301, 72), dtype, 1)
    toks = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=DEV)
    x = torch.empty((5, 72), dtype=torch.float32, device=DEV)
    o.embed(toks, table, x)
    assert torch.equal(x, table[toks.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,eps", [(72, 1e-5), (4096, 1e-6), (1000, 3e-3), (1001, 1e-5), (5120, 1e-5),
                                   (18000, 1e-5)])
def test_rmsnorm(dtype, H, eps):
    o = _ops(dtype)
    x = _rand((7, H), torch.float32, 2, 3.0)
    for wdt in (torch.float32, torch.bfloat16):
        w = (1 + 0.1 * _rand((H,), torch.float32, 3)).to(wdt)
        y = torch.empty((7, H), dtype=dtype, device=DEV)
        o.rmsnorm(x, w, eps, y)
        xd = x.double()
        ref = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + eps) * w.double()
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(y.double(), ref, rtol=tol, atol=tol)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    y = torch.empty((3, H), dtype=dtype, device=DEV)
    o.rmsnorm(x, w, eps, y, rows)
    full = torch.empty((7, H), dtype=dtype, device=DEV)
    o.rmsnorm(x, w, eps, full)
    assert torch.equal(y, full[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    o = _ops(dtype)
    gu = _rand((5, 2 * 177), torch.float32, 4, 3.0)
    out = torch.empty((5, 177), dtype=dtype, device=DEV)
    o.silu_mul(gu, out)
    g, u = gu[:, :177].double(), gu[:, 177:].double()
    ref = g / (1 + torch.exp(-g)) * u
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert torch.allclose(out.double(), ref, rtol=tol, atol=tol)


# ---------------------------------------------------------------------------
# matrix products on CUDA cores: every mode, skinny and tiled, odd sizes
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 50, 33), (3, 129, 72), (8, 64, 4096), (9, 65, 100),
                                   (70, 200, 177), (130, 31, 64)])
def test_gemm_generic(dtype, M, N, K):
    from torchless_rs_b200.csrc import ops
    o = _ops(dtype)
    a = _rand((M, K), dtype, 5)
    w = _rand((2 * N, K), dtype, 6, 1.0 / math.sqrt(K))   # products of size ~1
    ad, wd = a.double(), w.double()
    ref = ad @ wd[:N].T
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    c = torch.empty((M, N), dtype=torch.float32, device=DEV)
    o.gemm_generic(a, w[:N], c, ops.MODE_STORE_F32)
    assert torch.allclose(c.double(), ref, rtol=1e-5, atol=1e-4)
    base = _rand((M, N), torch.float32, 7)
    c2 = base.clone()
    o.gemm_generic(a, w[:N], c2, ops.MODE_ACCUM_F32)
    assert torch.allclose(c2.double(), base.double() + ref, rtol=1e-5, atol=1e-4)
    c3 = torch.empty((M, N), dtype=dtype, device=DEV)
    o.gemm_generic(a, w[:N], c3, ops.MODE_STORE_ACT)
    assert torch.allclose(c3.double(), ref, **tol)
    c4 = torch.empty((M, N), dtype=dtype, device=DEV)
    o.gemm_generic(a, w, c4, ops.MODE_SWIGLU)
    up = ad @ wd[N:].T
    assert torch.allclose(c4.double(), ref / (1 + torch.exp(-ref)) * up, **tol)


# ---------------------------------------------------------------------------
# paged cache helpers and a plain attention reference
# ---------------------------------------------------------------------------
class Paged:
    """Dense keys and values of several sequences laid into shuffled cache pages."""

    def __init__(self, lens, nkv, hd, dtype, seed, poison=True):
        self.lens, self.nkv, self.hd = list(lens), nkv, hd
        B = len(lens)
        g = torch.Generator().manual_seed(seed)
        self.k = [torch.randn((n, nkv, hd), generator=g).to(dtype) for n in lens]
        self.v = [torch.randn((n, nkv, hd), generator=g).to(dtype) for n in lens]
        need = sum((n + PAGE - 1) // PAGE for n in lens)
        n_pages = need + 3
        perm = torch.randperm(n_pages, generator=g).tolist()
        width = max((n + PAGE - 1) // PAGE for n in lens) + 1
        self.n_slots = B + 2
        self.slots = torch.randperm(self.n_slots, generator=g).tolist()[:B]
        assert len(set(self.slots)) == B
        table = torch.full((self.n_slots, width), -1, dtype=torch.int32)
        fill = 1e4 if poison else 0.0   # unused rows hold large finite numbers
        kp = torch.full((n_pages, nkv, PAGE, hd), fill).to(dtype)
        vp = torch.full((n_pages, nkv, hd, PAGE), fill).to(dtype)
        it = iter(perm)
        for b, n in enumerate(lens):
            for j in range((n + PAGE - 1) // PAGE):
                p = next(it)
                table[self.slots[b], j] = p
                cnt = min(PAGE, n - j * PAGE)
                kp[p, :, :cnt, :] = self.k[b][j * PAGE:j * PAGE + cnt].permute(1, 0, 2)
                vp[p, :, :, :cnt] = self.v[b][j * PAGE:j * PAGE + cnt].permute(1, 2, 0)
        self.k_pages, self.v_pages = kp.to(DEV), vp.to(DEV)
        self.table = table.to(DEV)
        self.seq_slot = torch.tensor(self.slots, dtype=torch.int32, device=DEV)


def attention_reference(q, k, v, pos, window, scale):
    """q [nh, hd] at position `pos` over k, v [n, nkv, hd]; float64."""
    nh, hd = q.shape
    nkv = k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.empty((nh, hd), dtype=torch.float64)
    for h in range(nh):
        kk = k[lo:pos + 1, h // (nh // nkv)].double()
        vv = v[lo:pos + 1, h // (nh // nkv)].double()
        p = torch.softmax((kk @ q[h].double()) * scale, dim=0)
        out[h] = p @ vv
    return out


def _attn_tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 3, 48, None), (4, 1, 16, 7), (8, 8, 256, 100),
                                               (5, 5, 80, 64)])
def test_attention_generic(dtype, nh, nkv, hd, window):
    """Mixed batch: one sequence in prefill from 0, one continuing, one decoding."""
    o = _ops(dtype)
    lens = [70, 200, 131]
    new = [70, 5, 1]            # tokens of this step; the rest is already cached
    pc = Paged(lens, nkv, hd, dtype, 20 + hd)
    T = sum(new)
    q = _rand((T, nh * hd), dtype, 21)
    token_seq = torch.tensor(sum([[b] * n for b, n in enumerate(new)], []), dtype=torch.int32, device=DEV)
    token_pos = torch.tensor(sum([list(range(L - n, L)) for L, n in zip(lens, new)], []),
                             dtype=torch.int32, device=DEV)
    out = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    scale = 1 / math.sqrt(hd)
    o.attn_generic(q, pc.k_pages, pc.v_pages, out, token_pos, token_seq, pc.seq_slot, pc.table,
                   nh, nkv, hd, window, scale)
    got = out.cpu().double().view(T, nh, hd)
    qc = q.cpu().view(T, nh, hd)
    for t in range(T):
        b, pos = int(token_seq[t]), int(token_pos[t])
        ref = attention_reference(qc[t], pc.k[b], pc.v[b], pos, window, scale)
        assert torch.allclose(got[t], ref, **_attn_tol(dtype)), f"token {t} (seq {b}, pos {pos})"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style", [0, 1])
@pytest.mark.parametrize("nh,nkv,hd,lens,new", [(3, 2, 32, [66, 9], [66, 2]),
                                                (5, 2, 128, [200, 131, 40], [200, 31, 40]),
                                                (2, 1, 64, [300], [300]), (3, 3, 256, [260, 3], [260, 3]),
                                                (3, 2, 32, [290, 9], [280, 2]), (4, 2, 48, [290], [290])])
def test_rope_cache_write(dtype, style, nh, nkv, hd, lens, new):
    """Few tokens and many (the many-token kernel turns the values in shared memory), runs of
    positions that cross pages, and sequences that go on from an earlier step."""
    o = _ops(dtype)
    pc = Paged(lens, nkv, hd, dtype, 30, poison=False)
    T = sum(new)
    qkv = _rand((T, (nh + 2 * nkv) * hd), torch.float32, 31)
    token_seq = torch.tensor(sum([[b] * n for b, n in enumerate(new)], []), dtype=torch.int32, device=DEV)
    pos_list = sum([list(range(L - n, L)) for L, n in zip(lens, new)], [])
    token_pos = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    half = hd // 2
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(half, dtype=torch.float64) / half)).float().to(DEV)
    qo = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    kp, vp = torch.zeros_like(pc.k_pages), torch.zeros_like(pc.v_pages)
    o.rope_cache_write(qkv, qo, kp, vp, token_pos, token_seq, pc.seq_slot, pc.table, inv, style,
                       nh, nkv, hd)
    ang = torch.tensor(pos_list, dtype=torch.float32)[:, None] * inv.cpu()[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x = qkv.cpu().view(T, nh + 2 * nkv, hd)
    rot = x[:, :nh + nkv].clone()
    if style == 0:
        a, b = rot[..., :half].clone(), rot[..., half:].clone()
        rot[..., :half], rot[..., half:] = a * c - b * s, a * s + b * c
    else:
        a, b = rot[..., 0::2].clone(), rot[..., 1::2].clone()
        rot[..., 0::2], rot[..., 1::2] = a * c - b * s, a * s + b * c
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert torch.allclose(qo.cpu().float().view(T, nh, hd), rot[:, :nh], **tol)
    table = pc.table.cpu()
    for t in range(T):
        b, pos = int(token_seq[t]), pos_list[t]
        page = int(table[pc.slots[b], pos // PAGE])
        assert torch.allclose(kp[page, :, pos % PAGE, :].cpu().float(), rot[t, nh:], **tol)
        assert torch.allclose(vp[page, :, :, pos % PAGE].cpu().float(), x[t, nh + nkv:], **tol)
    # nothing else was written
    assert int((kp != 0).any(-1).sum()) <= T * nkv


@pytest.mark.parametrize("use_tma", [True, False])
@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, None), (8, 2, 128, 100), (4, 4, 64, 33),
                                               (12, 1, 32, None), (32, 8, 128, 4096), (10, 5, 64, 64),
                                               (12, 1, 128, 70)])
def test_attention_decode_bf16(nh, nkv, hd, window, use_tma):
    """Split-KV decode kernel: lengths around the 32-key groups and page borders, and
    every split count from one to more than there are groups."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    from torchless_rs_b200.parts.runtime import Workspace
    dtype = torch.bfloat16
    att = AttentionBf16.get(hd)
    lens = [1, 31, 32, 33, 64, 65, 127, 129, 300, 1000]
    pc = Paged(lens, nkv, hd, dtype, 40 + hd)
    B = len(lens)
    q = _rand((B, nh * hd), dtype, 41)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    ws = Workspace(torch.device(DEV))
    qc = q.cpu().view(B, nh, hd)
    refs = [attention_reference(qc[b], pc.k[b], pc.v[b], lens[b] - 1, window, scale) for b in range(B)]
    for n_splits in (1, 2, 3, 4, 7, 8, 40):
        out = torch.full((B, nh * hd), float("nan"), dtype=dtype, device=DEV)
        att.decode(q, pc.k_pages, pc.v_pages, out, seq_len, pc.seq_slot, pc.table, nh, nkv, window,
                   scale, n_splits, ws, use_tma=use_tma)
        got = out.cpu().double().view(B, nh, hd)
        for b in range(B):
            assert torch.allclose(got[b], refs[b], **_attn_tol(dtype)), \
                f"splits {n_splits} seq {b} (len {lens[b]})"
    if use_tma and hd % 64 == 0:
        # a block takes `quantum` pages whatever the sequence's length: long sequences use many of the
        # splits, short ones few (their other blocks write empty partial results); with too few
        # splits for the longest sequence the last block takes the rest
        for quantum, n_splits in ((1, 16), (2, 8), (5, 4), (3, 3), (16, 1), (7, 32)):
            out = torch.full((B, nh * hd), float("nan"), dtype=dtype, device=DEV)
            att.decode(q, pc.k_pages, pc.v_pages, out, seq_len, pc.seq_slot, pc.table, nh, nkv, window,
                       scale, n_splits, ws, quantum=quantum)
            got = out.cpu().double().view(B, nh, hd)
            for b in range(B):
                assert torch.allclose(got[b], refs[b], **_attn_tol(dtype)), \
                    f"quantum {quantum} splits {n_splits} seq {b} (len {lens[b]})"
    # the same bits every time
    first = None
    for _ in range(12):
        out = torch.full((B, nh * hd), float("nan"), dtype=dtype, device=DEV)
        att.decode(q, pc.k_pages, pc.v_pages, out, seq_len, pc.seq_slot, pc.table, nh, nkv, window,
                   scale, 7, ws, use_tma=use_tma)
        first = out.clone() if first is None else first
        assert torch.equal(out, first)
    assert att.take_error() == 0


@pytest.mark.parametrize("use_tma", [True, False])
def test_attention_decode_far_key_stands_out(use_tma):
    """Random keys give near-uniform weights, which would hide a key that is skipped
    or read from the wrong page.  Here one far key matches the query strongly, so the
    output must be that key's value; its place runs over group, page and window edges."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    from torchless_rs_b200.parts.runtime import Workspace
    nh, nkv, hd, n = 8, 2, 128, 700
    dtype = torch.bfloat16
    att = AttentionBf16.get(hd)
    ws = Workspace(torch.device(DEV))
    for window in (None, 300):
        lo = 0 if window is None else n - window
        for hot in (lo, lo + 1, lo + 31, lo + 32, 447, 448, 511, 512, n - 2, n - 1):
            pc = Paged([n], nkv, hd, dtype, 50, poison=True)
            q = _rand((1, nh * hd), dtype, 51)
            qh = q.view(nh, hd).float()
            # key `hot` of each kv head points along the mean query of its heads, times 4
            k_dense = pc.k[0].clone()
            for kvh in range(nkv):
                qm = qh[kvh * (nh // nkv):(kvh + 1) * (nh // nkv)].mean(0).cpu()
                k_dense[hot, kvh] = (qm * 4).to(dtype)
            page = int(pc.table[pc.slots[0], hot // PAGE])
            pc.k_pages[page, :, hot % PAGE, :] = k_dense[hot].to(DEV)
            pc.k[0] = k_dense
            seq_len = torch.tensor([n], dtype=torch.int32, device=DEV)
            out = torch.empty((1, nh * hd), dtype=dtype, device=DEV)
            scale = 1 / math.sqrt(hd)
            att.decode(q, pc.k_pages, pc.v_pages, out, seq_len, pc.seq_slot, pc.table, nh, nkv,
                       window, scale, 5, ws, use_tma=use_tma)
            ref = attention_reference(q.cpu().view(nh, hd), pc.k[0], pc.v[0], n - 1, window, scale)
            assert torch.allclose(out.cpu().double().view(nh, hd), ref, rtol=2e-2, atol=2e-2), \
                f"window {window} hot key {hot}"


# ---------------------------------------------------------------------------
# tensor-core matrix products (tcgen05): every mode, every token tile, K splits, tails
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 4096, 4096), (16, 200, 72), (17, 384, 1000),
                                   (33, 130, 64), (64, 6144, 512), (100, 256, 176), (129, 128, 192),
                                   (300, 520, 328), (2048, 512, 256), (257, 700, 520),
                                   (1000, 2500, 136), (2048, 4096, 512), (1024, 5000, 2048),
                                   (100, 512, 4096), (200, 384, 2048), (300, 640, 4096),
                                   (300, 4096, 1024), (130, 6100, 768), (70, 4096, 4096),
                                   (300, 256, 14336), (200, 384, 8192), (513, 384, 256), (140, 256, 512),
                                   # K in 6, 5 and 3 splits (40, 48 and 80 tiles of 128 rows), and 129 to 256 tokens on single SMs
                                   (8, 5120, 4096), (3, 6144, 1280), (40, 6100, 1000), (12, 10240, 1024), (200, 4096, 4096),
                                   # 24 token tiles and more: weight strips in groups of 8 (3 strips; 8 + 1; 8 + 8 + 4 with a ragged edge)
                                   (6200, 520, 328), (8192, 2304, 256), (6150, 5000, 136)])
def test_gemm_tensor_core(M, N, K):
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16
    g = GemmBf16.get()
    dtype = torch.bfloat16
    a = _rand((M, K), dtype, 80)
    w = _rand((2 * N, K), dtype, 81, 1.0 / math.sqrt(K))
    ad, wd = a.double(), w.double()
    ref = ad @ wd[:N].T
    up = ad @ wd[N:].T
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    assert g.run(a, w[:N], c, 0)
    assert torch.allclose(c.double(), ref, rtol=1e-4, atol=1e-4), f"store: {(c.double()-ref).abs().max()}"
    base = _rand((M, N), torch.float32, 82)
    c2 = base.clone()
    assert g.run(a, w[:N], c2, 1)
    assert torch.allclose(c2.double(), base.double() + ref, rtol=1e-4, atol=1e-4)
    c3 = torch.empty((M, N), dtype=dtype, device=DEV)
    assert g.run(a, w[:N], c3, 3)
    assert torch.allclose(c3.double(), ref, rtol=1e-2, atol=1e-2)
    c4 = torch.empty((M, N), dtype=dtype, device=DEV)
    assert g.run(a, w, c4, 2)
    assert torch.allclose(c4.double(), ref / (1 + torch.exp(-ref)) * up, rtol=1e-2, atol=1e-2)
    # a second run gives the same bits (K splits are added in a fixed order)
    c5 = torch.empty_like(c)
    assert g.run(a, w[:N], c5, 0)
    assert torch.equal(c, c5)
    assert g.take_error() == 0


@pytest.mark.parametrize("M,N,K", [(300, 4096, 14336), (140, 1024, 8192), (2048, 1024, 1024), (8, 4096, 4096)])
def test_gemm_tensor_core_back_to_back(M, N, K):
    """The same accumulating product many times in a row without a synchronisation between the
    launches, which overlap at their edges: the partial tiles and flags of a K split over pairs
    of SMs, and the cluster reductions of the few-token kernel, must not leak from one launch
    into the next."""
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16
    g = GemmBf16.get()
    a = _rand((M, K), torch.bfloat16, 300)
    ws = [_rand((N, K), torch.bfloat16, 301 + i, 1.0 / math.sqrt(K)) for i in range(3)]
    ref = sum(a.double() @ w.double().T for w in ws) * 6
    for trial in range(2):
        c = torch.zeros((M, N), dtype=torch.float32, device=DEV)
        for it in range(18):
            assert g.run(a, ws[it % 3], c, 1)
        assert torch.allclose(c.double(), ref, rtol=1e-3, atol=1e-3 * float(ref.abs().max())), f"trial {trial}"
    assert g.take_error() == 0


@pytest.mark.parametrize("variant", ["tc", "tma", "plain"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, None), (8, 2, 128, 100), (4, 4, 64, 33),
                                               (3, 1, 32, None), (6, 3, 64, 64)])
def test_attention_prefill_bf16(nh, nkv, hd, window, variant):
    """Tensor-core prefill kernel: sequences from scratch and continuing ones, lengths
    around the 16-query warps, the 64-query tiles and the 32-key groups."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    dtype = torch.bfloat16
    att = AttentionBf16.get(hd)
    lens = [1, 17, 64, 65, 200, 331, 150]
    new = [1, 17, 64, 65, 200, 131, 1]      # the last two continue an existing sequence
    pc = Paged(lens, nkv, hd, dtype, 90 + hd)
    B, T = len(lens), sum(new)
    q = _rand((T, nh * hd), dtype, 91)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    scale = 1 / math.sqrt(hd)
    att.prefill(q, pc.k_pages, pc.v_pages, out, seq_start, seq_len, pc.seq_slot, pc.table, B,
                max(new), nh, nkv, window, scale, variant=variant)
    assert att.take_error() == 0
    got = out.cpu().double().view(T, nh, hd)
    qc = q.cpu().view(T, nh, hd)
    for b in range(B):
        for i in range(new[b]):
            tkn, pos = starts[b] + i, lens[b] - new[b] + i
            ref = attention_reference(qc[tkn], pc.k[b], pc.v[b], pos, window, scale)
            assert torch.allclose(got[tkn], ref, **_attn_tol(dtype)), f"seq {b} pos {pos}"


@pytest.mark.parametrize("nh,nkv,hd,window,lens,new", [
    (30, 3, 64, None, [399, 373, 159], [260, 333, 132]),
    (30, 3, 64, 100, [274, 319], [274, 157]),
    (20, 2, 128, None, [384, 369, 490], [243, 321, 393])])
def test_attention_prefill_tc_many_blocks_repeated(nh, nkv, hd, window, lens, new):
    """Many heads per key/value head, so that many blocks of the tensor-core prefill kernel run
    side by side on the same pages, and the same launch several times: a page's contribution
    once went missing now and then when a softmax warp rescaled the output while the product
    of the page before was still under way."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    att = AttentionBf16.get(hd)
    dtype = torch.bfloat16
    pc = Paged(lens, nkv, hd, dtype, 1000 + nh + hd)
    B, T, G = len(lens), sum(new), nh // nkv
    q = _rand((T, nh * hd), dtype, 1001)
    starts = [0]
    for n in new:
        starts.append(starts[-1] + n)
    seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    scale = 1 / math.sqrt(hd)
    ref = torch.empty((T, nh, hd), dtype=torch.float64, device=DEV)
    for b in range(B):
        k = pc.k[b].to(DEV).double().repeat_interleave(G, dim=1)     # [n, nh, hd]
        v = pc.v[b].to(DEV).double().repeat_interleave(G, dim=1)
        qq = q[starts[b]:starts[b + 1]].view(new[b], nh, hd).double()
        pos = torch.arange(lens[b] - new[b], lens[b], device=DEV)
        keys = torch.arange(lens[b], device=DEV)
        seen = keys[None, :] <= pos[:, None]
        if window:
            seen &= keys[None, :] > pos[:, None] - window
        sc = torch.einsum("qhd,khd->hqk", qq, k) * scale
        p = torch.softmax(sc.masked_fill(~seen[None], float("-inf")), -1)
        ref[starts[b]:starts[b + 1]] = torch.einsum("hqk,khd->qhd", p, v)
    for rep in range(8):
        out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        att.prefill(q, pc.k_pages, pc.v_pages, out, seq_start, seq_len, pc.seq_slot, pc.table, B,
                    max(new), nh, nkv, window, scale, variant="tc")
        assert att.take_error() == 0
        assert torch.allclose(out.double().view(T, nh, hd), ref, **_attn_tol(dtype)), f"repetition {rep}"


@pytest.mark.parametrize("kernel", ["prefill_bf16_tc", "prefill_bf16_tma", "prefill_bf16_plain", "generic_bf16",
                                    "generic_f32"])
def test_attention_far_key_stands_out_in_every_kernel(kernel):
    """The same idea as for the decode kernel, for the kernels that take many queries: one
    key far back matches the last queries strongly; with a window it sits on the window's
    first and last visible place and one place outside it."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    dtype = torch.float32 if kernel.endswith("f32") else torch.bfloat16
    nh, nkv, hd, n = 4, 2, 128 if kernel.startswith("prefill_bf16") else 48, 300
    scale = 1 / math.sqrt(hd)
    for window in (None, 100):
        last = n - 1
        lo = 0 if window is None else last - window + 1
        for hot in (lo - 1, lo, lo + 1, 191, 192, last - 1, last):
            if hot < 0:
                continue
            pc = Paged([n], nkv, hd, dtype, 77)
            q = _rand((n, nh * hd), dtype, 78)
            qh = q.view(n, nh, hd).float().cpu()
            k_dense = pc.k[0].clone()
            for kvh in range(nkv):      # key `hot` points along the last query's mean over its heads
                qm = qh[last, kvh * (nh // nkv):(kvh + 1) * (nh // nkv)].mean(0)
                k_dense[hot, kvh] = (qm * 4).to(dtype)
            page = int(pc.table[pc.slots[0], hot // PAGE])
            pc.k_pages[page, :, hot % PAGE, :] = k_dense[hot].to(DEV)
            pc.k[0] = k_dense
            out = torch.empty((n, nh * hd), dtype=dtype, device=DEV)
            pos = torch.arange(n, dtype=torch.int32, device=DEV)
            seq = torch.zeros(n, dtype=torch.int32, device=DEV)
            if kernel.startswith("prefill_bf16"):
                AttentionBf16.get(hd).prefill(
                    q, pc.k_pages, pc.v_pages, out, torch.tensor([0, n], dtype=torch.int32, device=DEV),
                    torch.tensor([n], dtype=torch.int32, device=DEV), pc.seq_slot, pc.table, 1, n, nh, nkv,
                    window, scale, variant=kernel.rsplit("_", 1)[1])
            else:
                _ops(dtype).attn_generic(q, pc.k_pages, pc.v_pages, out, pos, seq, pc.seq_slot, pc.table,
                                         nh, nkv, hd, window, scale)
            got = out.cpu().double().view(n, nh, hd)
            for p_ in (last, last - 1, max(hot, 0)):     # rows that see the hot key, or just miss it
                ref = attention_reference(q.cpu().view(n, nh, hd)[p_], pc.k[0], pc.v[0], p_, window, scale)
                assert torch.allclose(got[p_], ref, **_attn_tol(dtype)), f"{kernel} window {window} hot {hot} row {p_}"


@pytest.mark.parametrize("M", [1, 8, 64, 150, 300])
def test_gemm_folds_the_norm_between_two_products(M):
    """Producer: C += a @ w.T also leaves bf16(C * norm_weight) and per-tile sums of squares;
    consumer: a product on that, scaled by 1/rms, equals the product on the normed stream."""
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16
    from torchless_rs_b200.parts.linear import NormCarry
    g = GemmBf16.get()
    H, K, N2, eps = 256, 512, 384, 1e-5
    a = _rand((M, K), torch.bfloat16, 101)
    w = _rand((H, K), torch.bfloat16, 102, 1.0 / math.sqrt(K))
    nw = (1 + 0.1 * _rand((H,), torch.float32, 103)).to(torch.bfloat16)
    stream = _rand((M, H), torch.float32, 104)
    want_stream = stream.double() + a.double() @ w.double().T
    carry = NormCarry(torch.zeros((M, H), dtype=torch.bfloat16, device=DEV),
                      torch.zeros((M, (H + 127) // 128), dtype=torch.float32, device=DEV), H, eps)
    assert g.run(a, w, stream, 1, emit=(nw, carry))
    assert torch.allclose(stream.double(), want_stream, rtol=1e-4, atol=1e-4)
    if not carry.valid:       # many tokens: the kernel does not fold (it was measured to gain nothing)
        assert M > 128
        return
    assert torch.allclose(carry.xw.double(), want_stream * nw.double(), rtol=1e-2, atol=1e-2)
    assert torch.allclose(carry.ss.double().sum(1), (want_stream ** 2).sum(1), rtol=1e-4)
    w2 = _rand((2 * N2, H), torch.bfloat16, 105, 1.0 / math.sqrt(H))
    normed = want_stream / torch.sqrt((want_stream ** 2).mean(1, keepdim=True) + eps) * nw.double()
    ref = normed @ w2.double()[:N2].T
    up = normed @ w2.double()[N2:].T
    out = torch.empty((M, N2), dtype=torch.float32, device=DEV)
    assert g.run(carry.xw, w2[:N2], out, 0, scaled=carry)
    assert torch.allclose(out.double(), ref, rtol=2e-2, atol=2e-2)
    act = torch.empty((M, N2), dtype=torch.bfloat16, device=DEV)
    assert g.run(carry.xw, w2, act, 2, scaled=carry)
    assert torch.allclose(act.double(), ref / (1 + torch.exp(-ref)) * up, rtol=3e-2, atol=3e-2)
    assert g.take_error() == 0


@pytest.mark.parametrize("folded_norm", [False, True])
@pytest.mark.parametrize("style", [0, 1])
@pytest.mark.parametrize("nh,nkv,hd", [(8, 2, 128), (6, 3, 64), (12, 4, 32)])
def test_gemm_rotates_and_writes_the_cache_itself(nh, nkv, hd, style, folded_norm):
    """The q/k/v product of a few-token step with K split: its reduction rotates q and k at
    each token's position and writes q, the key pages and the (transposed) value pages; the
    32-bit q/k/v tensor is not written.  Positions cross page borders, sequences lie in
    shuffled slots and pages; with `folded_norm` the input is a prepared norm input whose
    1/rms scale the product applies before it rotates."""
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16, RopeArgs
    from torchless_rs_b200.parts.linear import NormCarry
    g = GemmBf16.get()
    dtype = torch.bfloat16
    lens, new = [66, 129, 5, 200], [3, 2, 5, 1]
    pc = Paged(lens, nkv, hd, dtype, 40, poison=False)
    T, K, N, eps = sum(new), 1024, (nh + 2 * nkv) * hd, 1e-5
    w = _rand((N, K), dtype, 41, 1.0 / math.sqrt(K))
    if folded_norm:
        stream = _rand((T, K), torch.float32, 42, 3.0)
        nw = 1 + 0.1 * _rand((K,), torch.float32, 43)
        a = (stream * nw).to(dtype)
        carry = NormCarry(a, stream.pow(2).view(T, K // 128, 128).sum(-1).contiguous(), K, eps)
        carry.valid = True
        rinv = 1.0 / torch.sqrt(stream.double().pow(2).mean(1, keepdim=True) + eps)
        qkv = (a.double() @ w.double().T) * rinv
    else:
        a, carry = _rand((T, K), dtype, 42), None
        qkv = a.double() @ w.double().T
    token_seq = torch.tensor(sum([[b] * n for b, n in enumerate(new)], []), dtype=torch.int32, device=DEV)
    pos_list = sum([list(range(L - n, L)) for L, n in zip(lens, new)], [])
    token_pos = torch.tensor(pos_list, dtype=torch.int32, device=DEV)
    half = hd // 2
    inv = (1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64),
                           torch.arange(half, dtype=torch.float64) / half)).float().to(DEV)
    qo = torch.zeros((T, nh * hd), dtype=dtype, device=DEV)
    kp, vp = torch.zeros_like(pc.k_pages), torch.zeros_like(pc.v_pages)
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    rope = RopeArgs(qo.data_ptr(), kp.data_ptr(), vp.data_ptr(), token_pos.data_ptr(), token_seq.data_ptr(),
                    pc.seq_slot.data_ptr(), pc.table.data_ptr(), inv.data_ptr(), pc.table.stride(0), style,
                    nh, nkv, hd)
    assert g.run(a, w, out, 0, scaled=carry, rope=rope)
    assert g.rope_applied, "the product did not take the rotation over: this path is not under test"
    assert g.take_error() == 0
    assert torch.isnan(out).all(), "the 32-bit q/k/v tensor was written although the product wrote q, k and v"
    ang = torch.tensor(pos_list, dtype=torch.float64)[:, None] * inv.cpu().double()[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x = qkv.cpu().view(T, nh + 2 * nkv, hd)
    rot = x[:, :nh + nkv].clone()
    if style == 0:
        p, q_ = rot[..., :half].clone(), rot[..., half:].clone()
        rot[..., :half], rot[..., half:] = p * c - q_ * s, p * s + q_ * c
    else:
        p, q_ = rot[..., 0::2].clone(), rot[..., 1::2].clone()
        rot[..., 0::2], rot[..., 1::2] = p * c - q_ * s, p * s + q_ * c
    tol = dict(rtol=1e-2, atol=1e-2)
    assert torch.allclose(qo.cpu().double().view(T, nh, hd), rot[:, :nh], **tol)
    table = pc.table.cpu()
    for t in range(T):
        b, pos = int(token_seq[t]), pos_list[t]
        page = int(table[pc.slots[b], pos // PAGE])
        assert torch.allclose(kp[page, :, pos % PAGE, :].cpu().double(), rot[t, nh:], **tol), f"key of token {t}"
        assert torch.allclose(vp[page, :, :, pos % PAGE].cpu().double(), x[t, nh + nkv:], **tol), f"value of token {t}"
    assert int((kp != 0).any(-1).sum()) <= T * nkv and int((vp != 0).any(-2).sum()) <= T * nkv, \
        "something besides the tokens' own rows was written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,integer", [((3, 5), False), ((1025, 1031), False), ((4097,), False),
                                           ((70, 9), True)])
def test_random_weights_same_bits_on_host_and_device(dtype, shape, integer):
    """The fill kernel and the host code draw the same bits for (seed, name, index): across a
    chunk border of the host code (1025 x 1031 > 2^20), for odd counts, vectors (norm
    weights: 1 + N(0, 0.1)) and integer tables."""
    from torchless_rs_b200.weights import TensorSpec, random_tensor
    spec = TensorSpec(shape, integer=integer)
    host = random_tensor("some.tensor.weight", spec, 12, dtype, "cpu")
    dev = random_tensor("some.tensor.weight", spec, 12, dtype, DEV)
    assert dev.is_cuda and dev.dtype == host.dtype and dev.shape == host.shape
    assert torch.equal(dev.cpu(), host)
    assert not torch.equal(host, random_tensor("some.tensor.weight", spec, 13, dtype, "cpu"))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("stored", [torch.float32, torch.bfloat16, torch.float16])
def test_weight_conversion_on_the_device(dtype, stored):
    """A stored tensor becomes the activation type where the kernels read it: widening is exact,
    rounding to bfloat16 goes to the nearest even; stacked matrices are filled block by block."""
    from torchless_rs_b200.parts.runtime import Runtime
    rt = Runtime(DEV, dtype)
    g = torch.Generator().manual_seed(7)
    a = (torch.randn((37, 72), generator=g) * 3).to(stored)
    b = (torch.randn((5, 72), generator=g) * 1e-3).to(stored)
    a[0, :4] = torch.tensor([0.0, -0.0, 65504.0 if stored == torch.float16 else 3e38, 1e-7]).to(stored)
    got = rt.stack([a, b])
    assert got.dtype == dtype and got.shape == (42, 72) and got.is_cuda
    assert torch.equal(got.cpu(), torch.cat([a, b]).to(dtype))
    assert torch.equal(rt.matrix(b).cpu(), b.to(dtype))
