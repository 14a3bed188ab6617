"""Each kernel alone against the plain reference of the same operation, at sizes other
than the tiny models': head sizes 16..256 in steps of 16, group sizes 1/3/4/5/8, widths
and vocabularies that are no power of two.  Where random data would hide a fault the
inputs are made so that it shows: one far key whose score stands out, a window's edge,
pages scattered over the pool."""
import math

import numpy as np
import pytest
import torch

import plain_llama as pl
from cpp_minilamma_b200.csrc import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
PAGE = K.PAGE


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


def attention_tol(dtype, impl, values):
    """The tensor-core attention kernels round the probabilities to bfloat16 before the P.V
    product (2^-9 relative each), so their output error is bounded by 2^-9 * sum_j p_j |v_j|
    <= 2^-9 * max|v|; the bound used is twice that.  The general kernels keep P in float32."""
    if dtype == torch.bfloat16 and impl == "tensor_core":
        return dict(rtol=1.6e-2, atol=2.0 ** -8 * float(np.abs(values).max()))
    return tol(dtype)


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def as64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 104, 4096])  # 104, 4096: the bfloat16 table's rows are read in 16-byte words
def test_embedding(dtype, width):
    table = rnd((1000, width), dtype, 1)
    tokens = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32)
    out = torch.empty((5, width), dtype=torch.float32, device=DEV)
    K.embedding(tokens.to(DEV), table.to(DEV), out)
    np.testing.assert_array_equal(out.cpu().numpy(), pl.embedding(as64(table), tokens.numpy()).astype(np.float32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [100, 1000, 4096, 13000])
def test_add_rmsnorm(dtype, width):
    rows, eps = 7, 3e-4
    x = rnd((rows, width), torch.float32, 2, 3.0)
    delta = rnd((rows, width), dtype, 3)
    w = 1 + 0.1 * rnd((width,), torch.float32, 4)
    xd, out = x.to(DEV), torch.empty((rows, width), dtype=dtype, device=DEV)
    K.add_rmsnorm(xd, delta.to(DEV), w.to(DEV), out, eps)
    summed = as64(x) + as64(delta)
    np.testing.assert_allclose(xd.cpu().numpy(), summed, rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(as64(out), pl.rms_norm(summed, as64(w), eps), **tol(dtype))
    # no delta; gathered rows leave x alone
    x2 = x.to(DEV)
    pick = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty((3, width), dtype=dtype, device=DEV)
    K.add_rmsnorm(x2, delta.to(DEV), w.to(DEV), out2, eps, rows=pick)
    np.testing.assert_array_equal(x2.cpu().numpy(), x.numpy())
    np.testing.assert_allclose(as64(out2), pl.rms_norm(summed[[6, 0, 3]], as64(w), eps), **tol(dtype))
    out3 = torch.empty((rows, width), dtype=dtype, device=DEV)
    K.add_rmsnorm(x2, None, w.to(DEV), out3, eps)
    np.testing.assert_allclose(as64(out3), pl.rms_norm(as64(x), as64(w), eps), **tol(dtype))


def test_rmsnorm_is_reproducible():
    x = rnd((5, 5000), torch.float32, 5).to(DEV)
    w = torch.ones(5000, device=DEV)
    a, b = torch.empty_like(x), torch.empty_like(x)
    K.add_rmsnorm(x, None, w, a, 1e-5)
    K.add_rmsnorm(x, None, w, b, 1e-5)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,block", [(250, 0), (176, 8), (1000, 8)])
def test_swiglu(dtype, inter, block):
    rows = 5
    gate, up = rnd((rows, inter), dtype, 6, 2.0), rnd((rows, inter), dtype, 7)
    if block:
        gu = torch.stack([gate.view(rows, inter // block, block), up.view(rows, inter // block, block)], dim=2)
        gu = gu.reshape(rows, 2 * inter)
    else:
        gu = torch.cat([gate, up], dim=1)
    out = torch.empty((rows, inter), dtype=dtype, device=DEV)
    K.swiglu(gu.contiguous().to(DEV), out, block)
    np.testing.assert_allclose(as64(out), pl.swiglu(as64(gate), as64(up)), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_cast_and_bias(dtype):
    x = rnd((3, 333), torch.float32, 8)
    y = torch.empty((3, 333), dtype=torch.bfloat16, device=DEV)
    K.cast(x.to(DEV), y)
    assert torch.equal(y.cpu(), x.to(torch.bfloat16))
    z = torch.empty((3, 333), dtype=torch.float32, device=DEV)
    K.cast(y, z)
    assert torch.equal(z.cpu(), x.to(torch.bfloat16).float())
    a = rnd((4, 77), dtype, 9).to(DEV)
    bias = rnd((77,), torch.float32, 10)
    before = as64(a)
    K.add_bias(a, bias.to(DEV))
    np.testing.assert_allclose(as64(a), before + as64(bias), **tol(dtype))


# ------------------------------------------------------------------------------------ #
class PagedCase:
    """Sequences of given context lengths with k, v scattered over shuffled pages."""

    def __init__(self, ctx_lens, n_kv_heads, head_dim, dtype, seed, n_slots=None, spare_pages=3):
        rng = np.random.RandomState(seed)
        self.ctx_lens = list(ctx_lens)
        B = len(ctx_lens)
        n_slots = n_slots or B + 2
        blocks = [(c + PAGE - 1) // PAGE for c in ctx_lens]
        n_pages = sum(blocks) + spare_pages
        self.max_blocks = max(blocks) + 1
        order = rng.permutation(n_pages)
        self.slots = rng.permutation(n_slots)[:B]
        table = np.full((n_slots, self.max_blocks), -1, dtype=np.int32)
        # unused pages hold NaN so that a read beyond a sequence's length shows
        self.k_cache = torch.full((n_pages, n_kv_heads, PAGE, head_dim), float("nan"), dtype=dtype)
        self.v_cache = torch.full((n_pages, n_kv_heads, PAGE, head_dim), float("nan"), dtype=dtype)
        self.k, self.v = [], []
        at = 0
        for b, c in enumerate(ctx_lens):
            k = rnd((c, n_kv_heads, head_dim), dtype, seed * 100 + b)
            v = rnd((c, n_kv_heads, head_dim), dtype, seed * 100 + 50 + b)
            self.k.append(k)
            self.v.append(v)
            for blk in range(blocks[b]):
                page = int(order[at]); at += 1
                table[self.slots[b], blk] = page
                n = min(PAGE, c - blk * PAGE)
                self.k_cache[page, :, :n] = k[blk * PAGE:blk * PAGE + n].transpose(0, 1)
                self.v_cache[page, :, :n] = v[blk * PAGE:blk * PAGE + n].transpose(0, 1)
        self.table = torch.from_numpy(table)

    def write(self):
        """Push (possibly edited) self.k / self.v back into the pages."""
        table = self.table.numpy()
        for b, c in enumerate(self.ctx_lens):
            for blk in range((c + PAGE - 1) // PAGE):
                page = table[self.slots[b], blk]
                n = min(PAGE, c - blk * PAGE)
                self.k_cache[page, :, :n] = self.k[b][blk * PAGE:blk * PAGE + n].transpose(0, 1)
                self.v_cache[page, :, :n] = self.v[b][blk * PAGE:blk * PAGE + n].transpose(0, 1)

    def dev(self):
        return (self.k_cache.to(DEV), self.v_cache.to(DEV), torch.tensor(self.slots, dtype=torch.int32, device=DEV),
                torch.tensor(self.ctx_lens, dtype=torch.int32, device=DEV), self.table.to(DEV))


@pytest.fixture(params=["tma", "tma_global_merge", "tensor_core", "general"])
def decode_impl(request):
    """bfloat16 decode attention has two tensor-core kernels: the TMA-fed one (head sizes 64/128,
    needs arrival counters when the context is split; it merges the splits inside a thread-block
    cluster, or - second variant - through global memory) and the cp.async one (16 .. 256 in steps of 16); the
    general kernel must stay right at those sizes too."""
    K.USE_TENSOR_CORE_DECODE = request.param != "general"
    K.USE_TMA_DECODE = request.param.startswith("tma")
    K.USE_CLUSTER_MERGE = request.param == "tma"
    yield "general" if request.param == "general" else "tensor_core"
    K.USE_TENSOR_CORE_DECODE = True
    K.USE_TMA_DECODE = True
    K.USE_CLUSTER_MERGE = True


DECODE_SHAPES = [  # heads, kv heads, head_dim
    (4, 2, 16), (6, 1, 32), (3, 3, 48), (10, 2, 80), (32, 8, 128), (8, 1, 256), (16, 16, 64), (64, 2, 16),
    (40, 2, 64), (5, 5, 128)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hk,d", DECODE_SHAPES)
@pytest.mark.parametrize("splits", [1, 3, 8, 16, 20])  # 20: more than a cluster holds, merged through global memory
def test_attention_decode(dtype, hq, hk, d, splits, decode_impl):
    ctx = [1, 63, 64, 65, 300, 129]
    case = PagedCase(ctx, hk, d, dtype, seed=hq * 7 + d)
    q = rnd((len(ctx), hq, d), dtype, 11)
    kc, vc, slots, ctx_t, table = case.dev()
    out = torch.empty((len(ctx), hq * d), dtype=dtype, device=DEV)
    scratch = torch.empty(K.attention_decode_scratch_floats(len(ctx), hq, d, splits), dtype=torch.float32, device=DEV)
    K.attention_decode(q.reshape(len(ctx), hq * d).to(DEV), kc, vc, slots, ctx_t, table, scratch, out,
                       len(ctx), hq, hk, d, splits, 0, 1.0 / math.sqrt(d))
    for b, c in enumerate(ctx):
        ref = pl.causal_attention(as64(q[b:b + 1]), as64(case.k[b]), as64(case.v[b]), q_positions=[c - 1])
        np.testing.assert_allclose(as64(out[b]).reshape(hq, d), ref[0],
                                   **attention_tol(dtype, decode_impl, as64(case.v[b])), err_msg=f"seq {b} ctx {c}")
    # with arrival counters the last block of each group merges the splits itself; the counters
    # come back as zeros, so the same buffer serves the next launch
    counters = torch.zeros(len(ctx) * hk * (-(-(hq // hk) // 16)), dtype=torch.int32, device=DEV)
    for _ in range(2):
        merged = torch.full_like(out, float("nan"))
        K.attention_decode(q.reshape(len(ctx), hq * d).to(DEV), kc, vc, slots, ctx_t, table, scratch, merged,
                           len(ctx), hq, hk, d, splits, 0, 1.0 / math.sqrt(d), counters=counters)
        if K.USE_TMA_DECODE and dtype == torch.bfloat16 and d in (64, 128):
            # with counters the TMA-fed kernel ran, without them the cp.async kernel: two kernels with
            # their own order of sums, each held to the plain reference
            for b, c in enumerate(ctx):
                ref = pl.causal_attention(as64(q[b:b + 1]), as64(case.k[b]), as64(case.v[b]), q_positions=[c - 1])
                np.testing.assert_allclose(as64(merged[b]).reshape(hq, d), ref[0],
                                           **attention_tol(dtype, decode_impl, as64(case.v[b])), err_msg=f"seq {b} ctx {c}")
        else:  # the same kernel, merged by its last block instead of the combine kernel
            np.testing.assert_allclose(as64(merged), as64(out), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5,
                                       atol=1e-3 if dtype == torch.bfloat16 else 1e-6)
        assert int(counters.abs().sum()) == 0
        assert K.take_device_error() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [0, 63, 64, 447, 448, 511, 700])
def test_attention_decode_far_key_stands_out(dtype, far, decode_impl):
    # one key among 701 gets a score far above the rest: the output must be its value
    hq, hk, d, c = 8, 2, 64, 701
    case = PagedCase([c, 5], hk, d, dtype, seed=far + 1)
    q = rnd((2, hq, d), dtype, 12, 0.1)
    for g in range(hk):
        direction = torch.zeros(d)
        direction[g] = 1.0
        case.k[0][far, g] = (direction * 40.0).to(dtype)
        q[0, g * (hq // hk):(g + 1) * (hq // hk)] = (direction * 40.0).to(dtype)
        case.v[0][far, g] = torch.full((d,), 3.0 + g).to(dtype)
    case.write()
    kc, vc, slots, ctx_t, table = case.dev()
    for splits in (1, 5):
        out = torch.empty((2, hq * d), dtype=dtype, device=DEV)
        scratch = torch.empty(K.attention_decode_scratch_floats(2, hq, d, splits), dtype=torch.float32, device=DEV)
        counters = torch.zeros(2 * hk, dtype=torch.int32, device=DEV)  # the tensor-core kernels merge their splits themselves
        K.attention_decode(q.reshape(2, hq * d).to(DEV), kc, vc, slots, ctx_t, table, scratch, out,
                           2, hq, hk, d, splits, 0, 1.0 / math.sqrt(d), counters=counters)
        got = as64(out[0]).reshape(hq, d)
        for h in range(hq):
            np.testing.assert_allclose(got[h], 3.0 + h // (hq // hk), rtol=1e-2, atol=1e-2)
        ref = pl.causal_attention(as64(q[0:1]), as64(case.k[0]), as64(case.v[0]), q_positions=[c - 1])
        np.testing.assert_allclose(got, ref[0], **attention_tol(dtype, decode_impl, as64(case.v[0])))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 5, 64, 100])
def test_attention_decode_window_edge(dtype, window, decode_impl):
    # the key just outside the window is made huge: it must not be seen; the one just inside is
    hq, hk, d = 4, 2, 64
    ctx = [300, 70, 3]
    case = PagedCase(ctx, hk, d, dtype, seed=window)
    q = rnd((3, hq, d), dtype, 13, 0.1)
    big = torch.zeros(d); big[0] = 30.0
    for b, c in enumerate(ctx):
        outside = c - 1 - window
        if outside >= 0:
            case.k[b][outside] = big.to(dtype)
            case.v[b][outside] = torch.full((hk, d), 1000.0).to(dtype)
    q[:, :, 0] = 30.0
    case.write()
    kc, vc, slots, ctx_t, table = case.dev()
    for splits in (1, 4):
        out = torch.empty((3, hq * d), dtype=dtype, device=DEV)
        scratch = torch.empty(K.attention_decode_scratch_floats(3, hq, d, splits), dtype=torch.float32, device=DEV)
        counters = torch.zeros(3 * hk, dtype=torch.int32, device=DEV)
        K.attention_decode(q.reshape(3, hq * d).to(DEV), kc, vc, slots, ctx_t, table, scratch, out,
                           3, hq, hk, d, splits, window, 1.0 / math.sqrt(d), counters=counters)
        for b, c in enumerate(ctx):
            ref = pl.causal_attention(as64(q[b:b + 1]), as64(case.k[b]), as64(case.v[b]), window=window,
                                      q_positions=[c - 1])
            np.testing.assert_allclose(as64(out[b]).reshape(hq, d), ref[0],
                                       **attention_tol(dtype, decode_impl, as64(case.v[b][max(0, c - window):])),
                                       err_msg=f"seq {b}")


@pytest.mark.parametrize("hq,hk,d", [(32, 8, 128), (8, 1, 256), (16, 16, 64), (40, 2, 64), (5, 5, 128)])
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("splits,window", [(1, 0), (3, 0), (2, 70)])
@pytest.mark.parametrize("encoded", [True, False])
@pytest.mark.parametrize("tma", ["cluster", "global", False])
def test_attention_decode_fused_with_rope_and_cache_write(hq, hk, d, interleaved, splits, window, encoded, tma, monkeypatch):
    """One launch (rotate q and k, write k and v, attend) against the separate kernels and the plain
    reference.  The slot of the new token holds NaN before the call, here and in the separate path."""
    monkeypatch.setattr(K, "USE_TMA_DECODE", bool(tma))   # the TMA-fed kernel (head sizes 64/128) or the cp.async one
    monkeypatch.setattr(K, "USE_CLUSTER_MERGE", tma == "cluster")  # its splits merged in a cluster or through global memory
    dtype = torch.bfloat16
    ctx = [1, 63, 64, 65, 300, 129]
    B = len(ctx)
    case = PagedCase(ctx, hk, d, dtype, seed=hq + d)
    width = (hq + 2 * hk) * d
    qkv = rnd((B, width), dtype, 21)
    inv = pl.rope_inverse_frequencies(d, 10000.0)
    ang = np.arange(400)[:, None] * inv[None, :]
    cos = torch.tensor(np.cos(ang), dtype=torch.float32, device=DEV) if encoded else None
    sin = torch.tensor(np.sin(ang), dtype=torch.float32, device=DEV) if encoded else None
    pos = np.array([c - 1 for c in ctx], dtype=np.int32)
    # the plain reference: the new token's k (rotated) and v replace the last cached position
    x = as64(qkv)
    rot = (lambda t: pl.apply_rope(t, pos, inv, interleaved)) if encoded else (lambda t: t)
    q_ref = as64(torch.tensor(rot(x[:, :hq * d].reshape(B, hq, d))).to(dtype))
    k_new = as64(torch.tensor(rot(x[:, hq * d:(hq + hk) * d].reshape(B, hk, d))).to(dtype))
    v_new = x[:, (hq + hk) * d:].reshape(B, hk, d)
    table = case.table.numpy()
    for b, c in enumerate(ctx):   # poison the new token's place
        page, off = table[case.slots[b], (c - 1) // PAGE], (c - 1) % PAGE
        case.k_cache[page, :, off] = float("nan")
        case.v_cache[page, :, off] = float("nan")
    kc, vc, slots, ctx_t, table_d = case.dev()
    scratch = torch.empty(K.attention_decode_scratch_floats(B, hq, d, splits), dtype=torch.float32, device=DEV)
    counters = torch.zeros(B * hk * (-(-(hq // hk) // 16)), dtype=torch.int32, device=DEV)
    out = torch.full((B, hq * d), float("nan"), dtype=dtype, device=DEV)
    K.attention_decode_fused(qkv.to(DEV), cos, sin, interleaved, True, kc, vc, slots, ctx_t, table_d, scratch, out,
                             B, hq, hk, d, splits, window, 1.0 / math.sqrt(d), counters=counters)
    assert int(counters.abs().sum()) == 0
    # separate kernels on a second copy of the cache
    kc2, vc2, _, _, _ = case.dev()
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    q2 = torch.empty((B, hq * d), dtype=dtype, device=DEV)
    K.rope_cache_write(qkv.to(DEV), None, cos, sin, i32(pos), i32(np.arange(B)), slots, table_d, q2, kc2, vc2, hq, hk, d,
                       interleaved)
    out2 = torch.empty_like(out)
    K.attention_decode(q2, kc2, vc2, slots, ctx_t, table_d, scratch, out2, B, hq, hk, d, splits, window,
                       1.0 / math.sqrt(d), counters=counters)
    same = lambda a, b: torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert same(kc, kc2) and same(vc, vc2)          # the cache, bit for bit (NaN places included)
    assert K.take_device_error() == 0
    for b, c in enumerate(ctx):
        k_all = np.concatenate([as64(case.k[b])[:c - 1], k_new[b:b + 1]])
        v_all = np.concatenate([as64(case.v[b])[:c - 1], v_new[b:b + 1]])
        ref = pl.causal_attention(q_ref[b:b + 1], k_all, v_all, q_positions=[c - 1], window=window or None)
        np.testing.assert_allclose(as64(out[b]).reshape(hq, d), ref[0], **attention_tol(dtype, "tensor_core", v_all),
                                   err_msg=f"seq {b} ctx {c}")
    np.testing.assert_allclose(as64(out), as64(out2), rtol=1.6e-2, atol=2.0 ** -8 * float(np.abs(v_new).max() + 4))


@pytest.mark.parametrize("hq,hk,d", [(32, 8, 128), (16, 16, 64), (40, 2, 64)])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("fused", [True, False])
def test_attention_decode_in_a_given_order(hq, hk, d, splits, fused):
    """The TMA-fed kernel starts the blocks of the sequences in the order it is given (longest first in the engine):
    whatever the order, every sequence gets its own result, bit for bit the one of the plain order."""
    dtype = torch.bfloat16
    ctx = [1, 63, 64, 65, 700, 129, 2, 300]
    B = len(ctx)
    case = PagedCase(ctx, hk, d, dtype, seed=hq + d + 5)
    qkv = rnd((B, (hq + 2 * hk) * d), dtype, 29)
    kc, vc, slots, ctx_t, table_d = case.dev()
    scratch = torch.empty(max(1, K.attention_decode_scratch_floats(B, hq, d, splits)), dtype=torch.float32, device=DEV)
    counters = torch.zeros(B * hk * (-(-(hq // hk) // 16)), dtype=torch.int32, device=DEV)
    outs = []
    for order in (None, sorted(range(B), key=lambda i: -ctx[i]), [3, 0, 7, 1, 6, 2, 5, 4]):
        order_t = None if order is None else torch.tensor(order, dtype=torch.int32, device=DEV)
        out = torch.full((B, hq * d), float("nan"), dtype=dtype, device=DEV)
        k2, v2 = kc.clone(), vc.clone()
        if fused:
            K.attention_decode_fused(qkv.to(DEV), None, None, False, True, k2, v2, slots, ctx_t, table_d, scratch, out,
                                     B, hq, hk, d, splits, 0, 1.0 / math.sqrt(d), counters=counters, order=order_t)
        else:
            K.attention_decode(qkv[:, :hq * d].contiguous().to(DEV), k2, v2, slots, ctx_t, table_d, scratch, out,
                               B, hq, hk, d, splits, 0, 1.0 / math.sqrt(d), counters=counters, order=order_t)
        assert int(counters.abs().sum()) == 0 and K.take_device_error() == 0
        outs.append(out)
    x = as64(qkv)
    for b, c in enumerate(ctx):
        k_all, v_all = as64(case.k[b]).copy(), as64(case.v[b]).copy()
        if fused:   # the step's own key and value take the last place
            k_all[c - 1] = x[b, hq * d:(hq + hk) * d].reshape(hk, d)
            v_all[c - 1] = x[b, (hq + hk) * d:].reshape(hk, d)
        ref = pl.causal_attention(x[b:b + 1, :hq * d].reshape(1, hq, d), k_all, v_all, q_positions=[c - 1])
        np.testing.assert_allclose(as64(outs[0][b]).reshape(hq, d), ref[0], **attention_tol(dtype, "tensor_core", v_all),
                                   err_msg=f"seq {b} ctx {c}")
    same = lambda a, b: torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert same(outs[0], outs[1]) and same(outs[0], outs[2])
    with pytest.raises(K.KernelError):
        K.attention_decode(qkv[:, :hq * d].contiguous().to(DEV), kc, vc, slots, ctx_t, table_d, scratch, outs[0], B, hq, hk, d,
                           splits, 0, 1.0 / math.sqrt(d), counters=counters,
                           order=torch.zeros(B - 1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("hq,hk,d", [(32, 8, 128), (16, 16, 64), (40, 2, 64)])
@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("window", [0, 200])
def test_attention_decode_from_a_work_list(hq, hk, d, fused, window):
    """The TMA-fed kernel's launch as a list of (sequence, split) pairs: a sequence of 2,000 keys in 12 blocks and
    one of 700 in 3 beside short ones in one block each, the pairs in any order with unused places between
    them; every sequence against the plain reference, and twice over so that the counters are seen to come
    back as zeros."""
    dtype = torch.bfloat16
    ctx = [1, 63, 2000, 65, 700, 129, 2, 300]
    cuts = [1, 1, 12, 1, 3, 2, 1, 1] if not window else [1, 1, 4, 1, 2, 1, 1, 2]  # never more than a sequence has pages to read
    B = len(ctx)
    case = PagedCase(ctx, hk, d, dtype, seed=hq + d + 6)
    qkv = rnd((B, (hq + 2 * hk) * d), dtype, 31)
    kc, vc, slots, ctx_t, table_d = case.dev()
    most = K.WORK_LIST_MAX_SPLITS
    scratch = torch.empty(K.attention_decode_scratch_floats(B, hq, d, most), dtype=torch.float32, device=DEV)
    counters = torch.zeros(B * hk * (-(-(hq // hk) // 16)), dtype=torch.int32, device=DEV)
    pairs = [K.decode_work_entry(i, s, cuts[i]) for i in range(B) for s in range(cuts[i])]
    shuffled = list(np.random.RandomState(3).permutation(pairs))
    lists = [pairs + [-1] * 5, [-1, -1] + shuffled[:7] + [-1] + shuffled[7:] + [-1]]
    outs = []
    for work in lists:
        for _ in range(2):
            out = torch.full((B, hq * d), float("nan"), dtype=dtype, device=DEV)
            k2, v2 = kc.clone(), vc.clone()
            work_t = torch.tensor([int(w) for w in work], dtype=torch.int32, device=DEV)
            if fused:
                K.attention_decode_fused(qkv.to(DEV), None, None, False, True, k2, v2, slots, ctx_t, table_d, scratch, out,
                                         B, hq, hk, d, most, window, 1.0 / math.sqrt(d), counters=counters, work=work_t)
            else:
                K.attention_decode(qkv[:, :hq * d].contiguous().to(DEV), k2, v2, slots, ctx_t, table_d, scratch, out,
                                   B, hq, hk, d, most, window, 1.0 / math.sqrt(d), counters=counters, work=work_t)
            assert int(counters.abs().sum()) == 0 and K.take_device_error() == 0
            assert K.calls.get("attention_decode (TMA, work list)", 0) > 0
            outs.append(out)
    x = as64(qkv)
    for b, c in enumerate(ctx):
        k_all, v_all = as64(case.k[b]).copy(), as64(case.v[b]).copy()
        if fused:   # the step's own key and value take the last place
            k_all[c - 1] = x[b, hq * d:(hq + hk) * d].reshape(hk, d)
            v_all[c - 1] = x[b, (hq + hk) * d:].reshape(hk, d)
        ref = pl.causal_attention(x[b:b + 1, :hq * d].reshape(1, hq, d), k_all, v_all, q_positions=[c - 1],
                                  window=window or None)
        np.testing.assert_allclose(as64(outs[0][b]).reshape(hq, d), ref[0],
                                   **attention_tol(dtype, "tensor_core", v_all[max(0, c - window) if window else 0:]),
                                   err_msg=f"seq {b} ctx {c}")
    same = lambda a, b: torch.equal(a.view(torch.int16), b.view(torch.int16))
    assert all(same(outs[0], o) for o in outs[1:])  # the order of the pairs changes no bit
    with pytest.raises(K.KernelError, match="work list"):
        K.attention_decode(qkv[:, :hq * d].contiguous().to(DEV), kc, vc, slots, ctx_t, table_d, scratch, outs[0], B, hq, hk, d,
                           most, 0, 1.0 / math.sqrt(d), counters=counters,
                           work=torch.zeros(B - 1, dtype=torch.int32, device=DEV))


@pytest.fixture(params=["tcgen05", "tensor_core", "general"])
def prefill_impl(request):
    """tcgen05: the TMA/tensor-memory kernel (head sizes 64 and 128, else the next one);
    tensor_core: the mma.sync kernel; general: the kernel for every size and dtype."""
    K.USE_TENSOR_CORE_PREFILL = request.param != "general"
    K.USE_TCGEN05_PREFILL = request.param == "tcgen05"
    yield "general" if request.param == "general" else "tensor_core"
    K.USE_TENSOR_CORE_PREFILL = True
    K.USE_TCGEN05_PREFILL = True


def _prefill_tiles(q_lens, rows=64):
    tile_seq, tile_row0 = [], []
    for i, n in enumerate(q_lens):
        for r in range(0, n, rows):
            tile_seq.append(i)
            tile_row0.append(r)
    return tile_seq, tile_row0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hk,d", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (10, 2, 80), (8, 2, 128), (4, 1, 256),
                                      (6, 3, 64), (3, 1, 128), (2, 2, 64)])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_prefill(dtype, hq, hk, d, window, prefill_impl):
    # sequences that start at 0 and sequences that continue an existing context; tiles of 128 rows whose keys
    # fill one, two, three and five pages
    ctx = [200, 1, 65, 130, 64, 330, 449]
    q_lens = [200, 1, 3, 66, 64, 129, 300]
    case = PagedCase(ctx, hk, d, dtype, seed=d + hq)
    total = sum(q_lens)
    q = rnd((total, hq, d), dtype, 14)
    kc, vc, slots, ctx_t, table = case.dev()
    qstart = np.concatenate([[0], np.cumsum(q_lens)[:-1]]).astype(np.int32)
    tile_seq, tile_row0 = _prefill_tiles(q_lens)
    out = torch.empty((total, hq * d), dtype=dtype, device=DEV)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    # with the list of 128-row tiles where the window is off (the tcgen05 kernel takes either list)
    wide = None if window else tuple(i32(a) for a in _prefill_tiles(q_lens, 128))
    K.attention_prefill(q.reshape(total, hq * d).to(DEV), kc, vc, slots, ctx_t, i32(qstart), i32(q_lens),
                        i32(tile_seq), i32(tile_row0), table, out, len(tile_seq), hq, hk, d, window,
                        1.0 / math.sqrt(d), wide_tiles=wide)
    got = as64(out).reshape(total, hq, d)
    for b, (c, n) in enumerate(zip(ctx, q_lens)):
        rows = slice(qstart[b], qstart[b] + n)
        ref = pl.causal_attention(as64(q[rows]), as64(case.k[b]), as64(case.v[b]), window=window or None,
                                  q_positions=list(range(c - n, c)))
        np.testing.assert_allclose(got[rows], ref, **attention_tol(dtype, prefill_impl, as64(case.v[b])),
                                   err_msg=f"seq {b}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_prefill_far_key_stands_out(dtype, prefill_impl):
    hq, hk, d, c = 4, 2, 64, 520
    case = PagedCase([c], hk, d, dtype, seed=99)
    q = rnd((c, hq, d), dtype, 15, 0.1)
    far = 70
    direction = torch.zeros(d); direction[3] = 40.0
    case.k[0][far] = direction.to(dtype)
    case.v[0][far] = torch.full((hk, d), 7.0).to(dtype)
    q[:, :, :] = (direction * 1.0).to(dtype)
    case.write()
    kc, vc, slots, ctx_t, table = case.dev()
    tile_seq, tile_row0 = _prefill_tiles([c])
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    out = torch.empty((c, hq * d), dtype=dtype, device=DEV)
    K.attention_prefill(q.reshape(c, hq * d).to(DEV), kc, vc, slots, ctx_t, i32([0]), i32([c]), i32(tile_seq),
                        i32(tile_row0), table, out, len(tile_seq), hq, hk, d, 0, 1.0 / math.sqrt(d))
    got = as64(out).reshape(c, hq, d)
    np.testing.assert_allclose(got[far:], 7.0, rtol=1e-2, atol=1e-2)   # every query from `far` on sees it
    ref = pl.causal_attention(as64(q), as64(case.k[0]), as64(case.v[0]))
    np.testing.assert_allclose(got, ref, **attention_tol(dtype, prefill_impl, as64(case.v[0])))


EVERY_HEAD_SIZE = [(4, 2, 16), (6, 1, 32), (3, 3, 48), (16, 16, 64), (10, 2, 80), (6, 2, 96), (4, 4, 112), (32, 8, 128),
                   (3, 1, 144), (8, 2, 160), (34, 2, 176), (6, 3, 192), (4, 2, 208), (2, 2, 224), (5, 1, 240), (8, 1, 256)]


@pytest.mark.parametrize("hq,hk,d", EVERY_HEAD_SIZE)
@pytest.mark.parametrize("splits", [1, 3])
def test_attention_decode_on_tensor_cores_at_every_head_size(hq, hk, d, splits, monkeypatch):
    """The cp.async / mma.sync decode kernel takes head sizes 16 .. 256 in steps of 16: a warp owns whole
    8-column tiles of the output, and where the head's tiles do not divide by four the last warps own fewer
    (34 heads on 2 kv heads: two chunks of 16 heads and one of 1)."""
    monkeypatch.setattr(K, "USE_TMA_DECODE", False)
    test_attention_decode(torch.bfloat16, hq, hk, d, splits, "tensor_core")


@pytest.mark.parametrize("hq,hk,d", EVERY_HEAD_SIZE)
@pytest.mark.parametrize("interleaved", [True, False])
def test_attention_decode_fused_at_every_head_size(hq, hk, d, interleaved, monkeypatch):
    """The fused launch rotates the queries in their fragment registers; with pairs (i, i + d/2) the partner
    of a column lies d/2 further, which is a whole number of 16-column steps only when d is a multiple of 32."""
    test_attention_decode_fused_with_rope_and_cache_write(hq, hk, d, interleaved, 3, 0, True, False, monkeypatch)
    test_attention_decode_fused_with_rope_and_cache_write(hq, hk, d, interleaved, 2, 70, True, False, monkeypatch)


@pytest.mark.parametrize("hq,hk,d", EVERY_HEAD_SIZE)
@pytest.mark.parametrize("window", [0, 70])
def test_attention_prefill_on_tensor_cores_at_every_head_size(hq, hk, d, window, monkeypatch):
    """The mma.sync prefill kernel at head sizes 16 .. 256 (fewer blocks per multiprocessor above 128)."""
    monkeypatch.setattr(K, "USE_TCGEN05_PREFILL", False)
    test_attention_prefill(torch.bfloat16, hq, hk, d, window, "tensor_core")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("hq,hk,d", [(4, 2, 16), (3, 3, 48), (8, 2, 128)])
def test_rope_cache_write(dtype, interleaved, hq, hk, d):
    max_pos = 400
    inv = pl.rope_inverse_frequencies(d, 10000.0)
    ang = np.arange(max_pos)[:, None] * inv[None, :]
    cos, sin = torch.tensor(np.cos(ang), dtype=torch.float32), torch.tensor(np.sin(ang), dtype=torch.float32)
    starts, lens = [0, 63, 130], [5, 3, 70]   # tokens land on page edges
    ctx = [s + n for s, n in zip(starts, lens)]
    case = PagedCase(ctx, hk, d, dtype, seed=3)
    T = sum(lens)
    width = (hq + 2 * hk) * d
    qkv = rnd((T, width), dtype, 16)
    bias = rnd((width,), torch.float32, 17, 0.5)
    tok_pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)]).astype(np.int32)
    tok_seq = np.repeat(np.arange(3), lens).astype(np.int32)
    kc, vc, slots, _, table = case.dev()
    k_before, v_before = kc.clone(), vc.clone()
    q_out = torch.empty((T, hq * d), dtype=dtype, device=DEV)
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    K.rope_cache_write(qkv.to(DEV), bias.to(DEV), cos.to(DEV), sin.to(DEV), i32(tok_pos), i32(tok_seq), slots, table,
                       q_out, kc, vc, hq, hk, d, interleaved)
    x = as64(qkv) + as64(bias)
    q_ref = pl.apply_rope(x[:, :hq * d].reshape(T, hq, d), tok_pos, inv, interleaved)
    k_ref = pl.apply_rope(x[:, hq * d:(hq + hk) * d].reshape(T, hk, d), tok_pos, inv, interleaved)
    v_ref = x[:, (hq + hk) * d:].reshape(T, hk, d)
    np.testing.assert_allclose(as64(q_out).reshape(T, hq, d), q_ref, **tol(dtype))
    touched = torch.zeros(kc.shape[:1] + kc.shape[2:3], dtype=torch.bool)
    tab = case.table.numpy()
    for t in range(T):
        page, off = tab[case.slots[tok_seq[t]], tok_pos[t] // PAGE], tok_pos[t] % PAGE
        touched[page, off] = True
        np.testing.assert_allclose(as64(kc[page, :, off]), k_ref[t], **tol(dtype))
        np.testing.assert_allclose(as64(vc[page, :, off]), v_ref[t], **tol(dtype))
    # every other row of the cache is untouched, bit for bit
    same = lambda a, b: torch.equal(a.view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                                    b.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    keep = ~touched.to(DEV)
    assert same(kc.transpose(1, 2)[keep], k_before.transpose(1, 2)[keep])
    assert same(vc.transpose(1, 2)[keep], v_before.transpose(1, 2)[keep])


# ------------------------------------------------------------------------------------ #
@pytest.mark.parametrize("vocab", [1000, 50257, 128256])  # one block per row; a cluster per row, scalar and 16-byte loads
def test_argmax_first_of_ties_and_status(vocab):
    logits = rnd((6, vocab), torch.float32, 18)
    logits[0, 100] = logits[0, vocab - 300] = 9.0    # tie, far apart: the lower id wins (src/sampler.cc:31-41)
    logits[1] = 0.0                                   # all equal: id 0
    logits[2, vocab - 1] = 12.0
    logits[3, 7] = float("nan")
    logits[4, 0] = 20.0
    tokens = torch.empty(6, dtype=torch.int32, device=DEV)
    status = torch.empty(6, dtype=torch.int32, device=DEV)
    K.argmax(logits.to(DEV), tokens, status)
    got = tokens.cpu().tolist()
    assert got[0] == 100 and got[1] == 0 and got[2] == vocab - 1 and got[4] == 0
    assert got[5] == pl.greedy(logits[5].numpy())
    assert status.cpu().tolist() == [0, 0, 0, 1, 0, 0]


def _cdf_interval_ok(logits, temperature, top_k, u, token, slack=1e-4):
    """The token's slice of the cumulative distribution contains u (with float32 slack)."""
    logits = logits.astype(np.float64)
    ids = np.arange(len(logits))
    if top_k:
        ids = np.lexsort((ids, -logits))[:top_k]
    w = np.exp((logits[ids] - logits[ids].max()) / temperature)
    cdf = np.cumsum(w) / w.sum()
    where = np.nonzero(ids == token)[0]
    if len(where) == 0:
        return False
    i = int(where[0])
    lo = cdf[i - 1] if i else 0.0
    return lo - slack <= u <= cdf[i] + slack


# from 8,192 logits on a cluster of eight blocks shares a row, 16, 32 or 64 logits a thread; 9,001 and 151,937 are
# read with 4-byte loads
@pytest.mark.parametrize("vocab", [131, 1000, 9001, 50257, 128256, 151937])
@pytest.mark.parametrize("top_k", [0, 2, 40, 1000, 1024])
def test_sampling_follows_the_plain_rule(vocab, top_k):
    if top_k > vocab:
        top_k = vocab
    rows, temperature, seed = 48, 0.8, 1234
    logits = rnd((rows, vocab), torch.float32, 19, 3.0)
    logits[0, :10] = 5.0  # ties inside the kept set
    request = torch.arange(rows, dtype=torch.int32)
    step = (torch.arange(rows, dtype=torch.int32) * 7) % 13
    tokens = torch.empty(rows, dtype=torch.int32, device=DEV)
    status = torch.empty(rows, dtype=torch.int32, device=DEV)
    K.sample(logits.to(DEV), temperature, top_k, seed, request.to(DEV), step.to(DEV), tokens, status)
    again = torch.empty_like(tokens)
    K.sample(logits.to(DEV), temperature, top_k, seed, request.to(DEV), step.to(DEV), again, status)
    assert torch.equal(tokens, again)  # seeded: reproducible
    assert status.cpu().tolist() == [0] * rows
    exact = 0
    for r in range(rows):
        u = float(pl.uniform_from_counter(seed, int(request[r]), int(step[r])))
        token = int(tokens[r])
        assert _cdf_interval_ok(logits[r].numpy(), temperature, top_k, u, token), f"row {r}: token {token}, u {u}"
        exact += token == pl.sample(logits[r].numpy(), temperature, top_k, u)
        if vocab > 50257 or top_k:
            # In float64 the token's slice holds u to within the rounding of a float32 sum taken as a tree (runs of
            # at most 64 terms, then scans: 64 * 2^-24 of the total).  Over a whole vocabulary of this size the plain
            # rule, which sums one float32 after the other as the reference does, is itself several ids off.
            assert _cdf_interval_ok(logits[r].numpy(), temperature, top_k, u, token, slack=64 * 2.0 ** -24), \
                f"row {r}: token {token}, u {u}"
    if vocab <= 50257 or top_k:
        assert exact >= rows - 2  # identical but for float32 summation order at an interval's edge


@pytest.mark.parametrize("vocab", [1000, 128256])
@pytest.mark.parametrize("top_k", [0, 40])
def test_sampling_status_reports_non_finite_logits(vocab, top_k):
    logits = rnd((5, vocab), torch.float32, 23, 2.0)
    logits[1, vocab - 1] = float("inf")
    logits[3, vocab // 2 + 3] = float("nan")
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    tokens, status = i32([0] * 5), i32([7] * 5)
    K.sample(logits.to(DEV), 0.9, top_k, 11, i32([0, 1, 2, 3, 4]), i32([0] * 5), tokens, status)
    assert status.cpu().tolist() == [0, 1, 0, 1, 0]
    assert all(0 <= t < vocab for t in tokens.cpu().tolist())
    # a flag that a kernel raised comes back in the status word of row 0, once
    K.raise_device_error(0b0101)
    K.sample(logits.to(DEV), 0.9, top_k, 11, i32([0, 1, 2, 3, 4]), i32([0] * 5), tokens, status)
    assert status.cpu().tolist() == [0x500, 1, 0, 1, 0]
    K.sample(logits.to(DEV), 0.9, top_k, 11, i32([0, 1, 2, 3, 4]), i32([0] * 5), tokens, status)
    assert status.cpu().tolist() == [0, 1, 0, 1, 0]
    assert K.take_device_error() == 0


@pytest.mark.parametrize("vocab,rows", [(300, 4000), (128256, 1500)])
def test_sampling_distribution(vocab, rows):
    # 4 candidates (the last of them the row's last logit), thousands of draws: frequencies follow softmax(l / T)
    temperature = 1.5
    base = torch.full((vocab,), -50.0)
    base[[3, 50, 51, vocab - 1]] = torch.tensor([1.0, 2.0, 0.0, 1.5])
    logits = base.repeat(rows, 1).contiguous()
    request = torch.arange(rows, dtype=torch.int32, device=DEV)
    step = torch.zeros(rows, dtype=torch.int32, device=DEV)
    tokens = torch.empty(rows, dtype=torch.int32, device=DEV)
    status = torch.empty(rows, dtype=torch.int32, device=DEV)
    for top_k in (0, 4):
        K.sample(logits.to(DEV), temperature, top_k, 7, request, step, tokens, status)
        counts = np.bincount(tokens.cpu().numpy(), minlength=vocab)
        p = np.exp(np.array([1.0, 2.0, 0.0, 1.5]) / temperature)
        p /= p.sum()
        assert counts[[3, 50, 51, vocab - 1]].sum() == rows
        np.testing.assert_allclose(counts[[3, 50, 51, vocab - 1]] / rows, p, atol=0.03 if rows >= 4000 else 0.045)


def test_kernels_refuse_bad_sizes():
    q = torch.zeros((1, 4 * 24), dtype=torch.float32, device=DEV)
    cache = torch.zeros((2, 2, PAGE, 24), dtype=torch.float32, device=DEV)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    with pytest.raises(K.KernelError, match="multiple of 16"):
        K.attention_decode(q, cache, cache, i32([0]), i32([1]), i32([[0]]), None, torch.empty_like(q), 1, 4, 2, 24,
                           1, 0, 1.0)
    with pytest.raises(K.KernelError, match="CUDA tensor"):
        K.argmax(torch.zeros((1, 8)), i32([0]), i32([0]))
    with pytest.raises(K.KernelError, match="top_k"):
        K.sample(torch.zeros((1, 5000), device=DEV), 1.0, 2000, 1, i32([0]), i32([0]), i32([0]), i32([0]))


# ------------------------------------------------------------------------------------ #
@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,k,ranks", [(16, 32, 1), (40, 64, 2), (4104, 4096, 0), (512, 14336, 8), (128, 4096, 4),
                                        (100, 224, 1)])
def test_linear_small(rows, n, k, ranks):
    x = rnd((rows, k), torch.bfloat16, 30)
    w = rnd((n, k), torch.bfloat16, 31, 0.05)
    bias = rnd((n,), torch.float32, 32)
    ref = as64(x) @ as64(w).T
    assert K.linear_small_supported(rows, n, k)
    for epilogue, dtype, b in ((K.EPI_BF16, torch.bfloat16, None), (K.EPI_F32, torch.float32, bias)):
        out = torch.full((rows, n), float("nan"), dtype=dtype, device=DEV)
        K.linear_small(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), out, epilogue, ranks)
        want = ref if b is None else ref + as64(b)
        if dtype == torch.float32:  # float32 accumulation of exact bfloat16 products
            np.testing.assert_allclose(as64(out), want, rtol=2e-5, atol=2e-5 * np.abs(want).max())
        else:
            np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
        again = torch.empty_like(out)
        K.linear_small(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), again, epilogue, ranks)
        assert torch.equal(out, again)  # fixed summation order


@pytest.mark.parametrize("rows", [1, 8, 13, 64])
@pytest.mark.parametrize("inter,k,ranks", [(176, 64, 1), (1000, 4096, 0), (64, 14336, 8)])
def test_linear_small_swiglu(rows, inter, k, ranks):
    gate = rnd((inter, k), torch.bfloat16, 33, 0.05)
    up = rnd((inter, k), torch.bfloat16, 34, 0.05)
    x = rnd((rows, k), torch.bfloat16, 35)
    fused = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear_small(x.to(DEV), fused.contiguous().to(DEV), None, out, K.EPI_SWIGLU, ranks)
    want = pl.swiglu(as64(x) @ as64(gate).T, as64(x) @ as64(up).T)
    np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())


def test_linear_small_refuses():
    assert not K.linear_small_supported(65, 4096, 4096)
    assert not K.linear_small_supported(8, 4096, 100)
    assert not K.linear_small_supported(8, 8, 64)
    with pytest.raises(K.KernelError, match="unsupported sizes"):
        K.linear_small(torch.zeros((2, 48), dtype=torch.bfloat16, device=DEV),
                       torch.zeros((16, 48), dtype=torch.bfloat16, device=DEV), None,
                       torch.zeros((2, 16), dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,k,ranks", [(16, 32, 1), (40, 64, 2), (4104, 4096, 0), (512, 14336, 8), (128, 4096, 4),
                                        (100, 224, 1), (7, 8, 1), (257, 200, 2), (1000, 1096, 0)])
def test_linear_tma(rows, n, k, ranks):
    # N that is no multiple of the 64-row tile, K that is no multiple of the 64-column stage:
    # the TMA unit fills what lies outside with zeros
    x = rnd((rows, k), torch.bfloat16, 40)
    w = rnd((n, k), torch.bfloat16, 41, 0.05)
    bias = rnd((n,), torch.float32, 42)
    ref = as64(x) @ as64(w).T
    assert K.linear_tma_supported(rows, n, k)
    for epilogue, dtype, b in ((K.EPI_BF16, torch.bfloat16, None), (K.EPI_F32, torch.float32, bias)):
        out = torch.full((rows, n), float("nan"), dtype=dtype, device=DEV)
        K.linear_tma(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), out, epilogue, ranks)
        want = ref if b is None else ref + as64(b)
        if dtype == torch.float32:
            np.testing.assert_allclose(as64(out), want, rtol=2e-5, atol=2e-5 * np.abs(want).max())
        else:
            np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
        again = torch.empty_like(out)
        K.linear_tma(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), again, epilogue, ranks)
        assert torch.equal(out, again)
    assert K.take_device_error() == 0


@pytest.mark.parametrize("rows", [1, 8, 13, 64])
@pytest.mark.parametrize("inter,k,ranks", [(176, 64, 1), (1000, 4096, 0), (64, 14336, 8), (40, 72, 1)])
def test_linear_tma_swiglu(rows, inter, k, ranks):
    gate = rnd((inter, k), torch.bfloat16, 43, 0.05)
    up = rnd((inter, k), torch.bfloat16, 44, 0.05)
    x = rnd((rows, k), torch.bfloat16, 45)
    fused = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear_tma(x.to(DEV), fused.contiguous().to(DEV), None, out, K.EPI_SWIGLU, ranks)
    want = pl.swiglu(as64(x) @ as64(gate).T, as64(x) @ as64(up).T)
    np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
    assert K.take_device_error() == 0


def test_linear_tma_refuses():
    assert not K.linear_tma_supported(65, 4096, 4096)
    assert not K.linear_tma_supported(8, 4096, 100)   # rows of 200 bytes: TMA needs multiples of 16
    with pytest.raises(K.KernelError, match="unsupported sizes"):
        K.linear_tma(torch.zeros((2, 12), dtype=torch.bfloat16, device=DEV),
                     torch.zeros((16, 12), dtype=torch.bfloat16, device=DEV), None,
                     torch.zeros((2, 16), dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("rows", [1, 3, 8, 13, 16, 17, 32, 33, 50, 64])
@pytest.mark.parametrize("n,k,ranks", [(16, 32, 1), (40, 64, 2), (4104, 4096, 0), (512, 14336, 8), (128, 4096, 4),
                                        (100, 224, 1), (7, 8, 1), (257, 200, 2), (1000, 1096, 0), (6144, 4096, 0),
                                        (6144, 4096, 4), (3072, 2048, 8)])
def test_linear_tc5(rows, n, k, ranks):
    # the tcgen05 / TMEM kernel: same contract as the TMA kernel, 16, 32 or 64 batch columns by the row count
    x = rnd((rows, k), torch.bfloat16, 50)
    w = rnd((n, k), torch.bfloat16, 51, 0.05)
    bias = rnd((n,), torch.float32, 52)
    ref = as64(x) @ as64(w).T
    assert K.linear_tc5_supported(rows, n, k)
    for epilogue, dtype, b in ((K.EPI_BF16, torch.bfloat16, None), (K.EPI_F32, torch.float32, bias)):
        out = torch.full((rows, n), float("nan"), dtype=dtype, device=DEV)
        K.linear_tc5(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), out, epilogue, ranks)
        want = ref if b is None else ref + as64(b)
        if dtype == torch.float32:
            np.testing.assert_allclose(as64(out), want, rtol=2e-5, atol=2e-5 * np.abs(want).max())
        else:
            np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
        again = torch.empty_like(out)
        K.linear_tc5(x.to(DEV), w.to(DEV), None if b is None else b.to(DEV), again, epilogue, ranks)
        assert torch.equal(out, again)
    assert K.take_device_error() == 0


@pytest.mark.parametrize("rows", [1, 8, 13, 16, 17, 32, 40, 64])
@pytest.mark.parametrize("inter,k,ranks", [(176, 64, 1), (1000, 4096, 0), (64, 14336, 8), (40, 72, 1)])
def test_linear_tc5_swiglu(rows, inter, k, ranks):
    gate = rnd((inter, k), torch.bfloat16, 53, 0.05)
    up = rnd((inter, k), torch.bfloat16, 54, 0.05)
    x = rnd((rows, k), torch.bfloat16, 55)
    fused = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.linear_tc5(x.to(DEV), fused.contiguous().to(DEV), None, out, K.EPI_SWIGLU, ranks)
    want = pl.swiglu(as64(x) @ as64(gate).T, as64(x) @ as64(up).T)
    np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
    assert K.take_device_error() == 0


# ---- a norm folded into the products around it ---------------------------------------- #
def _prenormed(rows, k, seed, eps):
    """A residual stream, the norm's weight, and what the residual epilogue leaves of them: the rows
    times the weight in bfloat16 and partial sums of squares per 16 columns."""
    stream = rnd((rows, k), torch.float32, seed, 3.0)
    weight = 1.0 + rnd((k,), torch.float32, seed + 1, 0.2)
    values = (stream * weight).to(torch.bfloat16)
    partials = -(-k // K.NORM_TILE)
    stride = partials + 3  # the stride may exceed the count; what lies beyond is not read
    sumsq = torch.full((rows, stride), float("nan"), dtype=torch.float32)
    padded = torch.zeros((rows, partials * K.NORM_TILE), dtype=torch.float64)
    padded[:, :k] = stream.double() ** 2
    sumsq[:, :partials] = padded.view(rows, partials, K.NORM_TILE).sum(-1).float()
    factor = 1.0 / np.sqrt((as64(stream) ** 2).mean(-1, keepdims=True) + eps)
    return stream, weight, values, K.RowNorm(sumsq.to(DEV), partials, eps), factor


@pytest.mark.parametrize("rows", [1, 3, 8, 13, 16, 17, 40, 64])
@pytest.mark.parametrize("n,k", [(48, 64), (4104, 4096), (100, 224), (6144, 4096), (512, 8192)])
@pytest.mark.parametrize("kind", ["direct", "tma", "tc5"])
def test_linear_finishes_the_norm_before_it(rows, n, k, kind):
    # the product of rows that lack their norm's factor, times the factor, against norm then product
    eps = 1e-5
    stream, weight, values, row_norm, factor = _prenormed(rows, k, 60, eps)
    w = rnd((n, k), torch.bfloat16, 62, 0.05)
    bias = rnd((n,), torch.float32, 63)
    run = {"direct": K.linear_small, "tma": K.linear_tma, "tc5": K.linear_tc5}[kind]
    if kind == "direct" and not K.linear_small_supported(rows, n, k):
        pytest.skip("the direct kernel does not take this shape")
    want = (as64(values) * factor) @ as64(w).T
    against_norm = pl.rms_norm(as64(stream), as64(weight), eps) @ as64(w).T
    np.testing.assert_allclose(want, against_norm, rtol=0, atol=8e-3 * np.abs(against_norm).max())
    out = torch.full((rows, n), float("nan"), dtype=torch.float32, device=DEV)
    run(values.to(DEV), w.to(DEV), bias.to(DEV), out, K.EPI_F32, 0, row_norm)
    np.testing.assert_allclose(as64(out), want + as64(bias), rtol=2e-5, atol=2e-5 * np.abs(want).max())
    out = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    run(values.to(DEV), w.to(DEV), None, out, K.EPI_BF16, 2 if k >= 4096 else 1, row_norm)
    np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
    assert K.take_device_error() == 0


@pytest.mark.parametrize("rows", [2, 8, 11])
@pytest.mark.parametrize("kind", ["direct", "tma", "tc5"])
def test_linear_swiglu_finishes_the_norm_before_it(rows, kind):
    inter, k, eps = 176, 320, 1e-6
    stream, weight, values, row_norm, factor = _prenormed(rows, k, 64, eps)
    gate = rnd((inter, k), torch.bfloat16, 66, 0.05)
    up = rnd((inter, k), torch.bfloat16, 67, 0.05)
    fused = torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)
    run = {"direct": K.linear_small, "tma": K.linear_tma, "tc5": K.linear_tc5}[kind]
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    run(values.to(DEV), fused.contiguous().to(DEV), None, out, K.EPI_SWIGLU, 0, row_norm)
    h = as64(values) * factor
    want = pl.swiglu(h @ as64(gate).T, h @ as64(up).T)
    np.testing.assert_allclose(as64(out), want, rtol=8e-3, atol=8e-3 * np.abs(want).max())
    assert K.take_device_error() == 0


@pytest.mark.parametrize("rows", [1, 3, 8, 13, 16, 17, 31, 32, 33, 64])
@pytest.mark.parametrize("n,k,ranks", [(48, 64, 1), (4096, 4096, 0), (100, 224, 1), (4096, 14336, 0), (520, 4096, 4),
                                        (2048, 8192, 8)])
@pytest.mark.parametrize("normed_input", [False, True])
@pytest.mark.parametrize("kind", ["direct", "tc5"])
def test_linear_adds_to_the_residual_and_starts_the_next_norm(rows, n, k, ranks, normed_input, kind):
    if kind == "direct" and rows > 16:
        pytest.skip("the direct kernel's residual epilogue takes at most 16 rows")
    run = {"direct": K.linear_small, "tc5": K.linear_tc5}[kind]
    eps = 1e-5
    if normed_input:
        _, _, x, row_norm, factor = _prenormed(rows, k, 70, eps)
    else:
        x, row_norm, factor = rnd((rows, k), torch.bfloat16, 70), None, 1.0
    w = rnd((n, k), torch.bfloat16, 72, 0.05)
    resid = rnd((rows, n), torch.float32, 73, 2.0)
    next_w = 1.0 + rnd((n,), torch.float32, 74, 0.2)
    tiles = -(-n // K.NORM_TILE)
    stride = tiles + 5
    resid_dev = resid.to(DEV)
    values = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    sumsq = torch.full((rows, stride), float("nan"), dtype=torch.float32, device=DEV)
    run(x.to(DEV), w.to(DEV), None, values, K.EPI_RESID, ranks, row_norm, K.ResidualOut(resid_dev, next_w.to(DEV), sumsq))
    want = as64(resid) + (as64(x) * factor) @ as64(w).T
    np.testing.assert_allclose(as64(resid_dev), want, rtol=2e-5, atol=2e-5 * np.abs(want).max())
    np.testing.assert_allclose(as64(values), want * as64(next_w), rtol=8e-3, atol=1e-3)
    # the partial sums are those of the stream as the kernel wrote it, and only the first `tiles` are written
    got = as64(resid_dev)
    padded = np.zeros((rows, tiles * K.NORM_TILE))
    padded[:, :n] = got ** 2
    np.testing.assert_allclose(as64(sumsq)[:, :tiles], padded.reshape(rows, tiles, K.NORM_TILE).sum(-1), rtol=1e-5)
    assert torch.isnan(sumsq[:, tiles:]).all()
    # the pair is a norm: values * factor from the sums is rms_norm(new stream) * next_w
    factor_out = 1.0 / np.sqrt(as64(sumsq)[:, :tiles].sum(-1, keepdims=True) / n + eps)
    normed = pl.rms_norm(got, as64(next_w), eps)
    np.testing.assert_allclose(as64(values) * factor_out, normed, rtol=8e-3, atol=1e-3)
    assert K.take_device_error() == 0


@pytest.mark.parametrize("rows,inter,k,block", [(1, 176, 64, 8), (17, 14336, 4096, 8), (64, 8192, 2048, 8), (40, 200, 96, 0)])
def test_swiglu_finishes_the_norm_before_the_product(rows, inter, k, block):
    # gate/up computed by a product that could not apply the rows' norm factors: the activation kernel does
    eps = 1e-5
    _, _, values, row_norm, factor = _prenormed(rows, k, 90, eps)
    gate = rnd((rows, inter), torch.bfloat16, 91, 2.0)   # stands for (x w_norm) . Wgate^T, not yet scaled
    up = rnd((rows, inter), torch.bfloat16, 92, 2.0)
    if block:
        gu = torch.stack([gate.view(rows, inter // 8, 8), up.view(rows, inter // 8, 8)], dim=2).reshape(rows, 2 * inter)
    else:
        gu = torch.cat([gate, up], dim=1)
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.swiglu(gu.contiguous().to(DEV), out, block, row_norm, k)
    want = pl.swiglu(as64(gate) * factor, as64(up) * factor)
    np.testing.assert_allclose(as64(out), want, rtol=1e-2, atol=1e-2 * np.abs(want).max())


def test_apply_row_norm():
    rows, k, eps = 5, 200, 1e-5
    _, _, values, row_norm, factor = _prenormed(rows, k, 80, eps)
    out = torch.full((rows, k), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.apply_row_norm(values.to(DEV), row_norm, out)
    np.testing.assert_allclose(as64(out), as64(values) * factor, rtol=4e-3, atol=1e-6)


def test_linear_small_residual_refuses():
    x = torch.zeros((17, 64), dtype=torch.bfloat16, device=DEV)
    w = torch.zeros((32, 64), dtype=torch.bfloat16, device=DEV)
    target = K.ResidualOut(torch.zeros((17, 32), device=DEV), torch.ones((32,), device=DEV), torch.zeros((17, 4), device=DEV))
    with pytest.raises(K.KernelError, match="at most 16 rows"):
        K.linear_small(x, w, None, torch.zeros((17, 32), dtype=torch.bfloat16, device=DEV), K.EPI_RESID, 0, None, target)
    with pytest.raises(K.KernelError, match="go together"):
        K.linear_small(x[:4], w, None, torch.zeros((4, 32), dtype=torch.bfloat16, device=DEV), K.EPI_RESID)
    short = K.ResidualOut(torch.zeros((4, 32), device=DEV), torch.ones((32,), device=DEV), torch.zeros((4, 1), device=DEV))
    with pytest.raises(K.KernelError, match="stride"):
        K.linear_small(x[:4], w, None, torch.zeros((4, 32), dtype=torch.bfloat16, device=DEV), K.EPI_RESID, 0, None, short)
