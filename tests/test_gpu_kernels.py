"""Each CUDA kernel alone against a plain float32 torch computation of the same operation, at sizes
other than the models' (odd widths, groups of 1 / 5 / 6, head sizes 16 / 48 / 128 / 256, pages that
are crossed, windows)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def K():
    from garlic_inference_b200.ops import kernels
    return kernels


def ulp_tol(dtype):
    # bfloat16: a result rounded once from float32 may differ by one step of 2^-8 relative
    return dict(rtol=2 ** -7, atol=1e-3) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-6)


# ------------------------------------------------------------------ row-wise kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(77, 100, generator=g, device=DEV).to(dtype)
    ids = torch.tensor([0, 76, 5, 5, 80, -1, 33], dtype=torch.int32, device=DEV)
    out = K().embedding(ids, table)
    assert out.dtype == torch.float32 and out.shape == (7, 100)
    ok = [0, 1, 2, 3, 6]
    assert torch.equal(out[ok], table[ids[ok].long()].float())
    assert float(out[4].abs().sum()) == 0 and float(out[5].abs().sum()) == 0      # ids outside the table


@pytest.mark.parametrize("act", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [48, 100, 1000, 4096])
def test_add_rmsnorm(act, wdt, dim):
    g = torch.Generator(device=DEV).manual_seed(dim)
    res = torch.randn(9, dim, generator=g, device=DEV) * 3
    delta = torch.randn(9, dim, generator=g, device=DEV).to(act)
    w = (1 + 0.3 * torch.randn(dim, generator=g, device=DEV)).to(wdt)
    eps = 3e-5

    def ref(s):
        return s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * w.float()

    r1 = res.clone()
    out = K().add_rmsnorm(delta, r1, w, eps, act)
    s = res + delta.float()
    assert torch.equal(r1, s), "the float32 sum goes back into the residual"
    torch.testing.assert_close(out.float(), ref(s).to(act).float(), **ulp_tol(act))
    r2 = res.clone()
    out = K().add_rmsnorm(None, r2, w, eps, act)
    assert torch.equal(r2, res)
    torch.testing.assert_close(out.float(), ref(res).to(act).float(), **ulp_tol(act))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    r3 = res.clone()
    out = K().add_rmsnorm(delta, r3, w, eps, act, rows=rows)
    assert torch.equal(r3, res), "gathered rows leave the residual alone"
    torch.testing.assert_close(out.float(), ref(s)[rows.long()].to(act).float(), **ulp_tol(act))


def test_add_rmsnorm_row_result_does_not_depend_on_the_batch():
    g = torch.Generator(device=DEV).manual_seed(1)
    res = torch.randn(33, 1536, generator=g, device=DEV)
    w = torch.randn(1536, generator=g, device=DEV)
    whole = K().add_rmsnorm(None, res.clone(), w, 1e-6, torch.float32)
    one = K().add_rmsnorm(None, res[17:18].clone(), w, 1e-6, torch.float32)
    assert torch.equal(whole[17:18], one)


@pytest.mark.parametrize("dtype,inter", [(torch.float32, 13), (torch.bfloat16, 13), (torch.bfloat16, 112)])
def test_swiglu(dtype, inter):
    g = torch.Generator(device=DEV).manual_seed(2)
    gu = (torch.randn(11, 2 * inter, generator=g, device=DEV) * 4).to(dtype)
    out = K().swiglu(gu)
    gate, up = gu[:, :inter].float(), gu[:, inter:].float()
    ref = (gate / (1 + torch.exp(-gate)) * up).to(dtype)
    torch.testing.assert_close(out.float(), ref.float(), **ulp_tol(dtype))


def test_cast_and_residual_add():
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(1001, generator=g, device=DEV)
    b = K().cast(x, torch.bfloat16)
    assert torch.equal(b, x.to(torch.bfloat16)) and torch.equal(K().cast(b, torch.float32), b.float())
    res = torch.randn(7, 143, generator=g, device=DEV)
    want = res + b[:1001].float().view(7, 143)
    K().residual_add(b.view(7, 143), res)
    assert torch.equal(res, want)


# ------------------------------------------------------------------ products
@pytest.mark.parametrize("m,n,k", [(1, 130, 50), (70, 130, 50), (64, 64, 16), (129, 65, 257)])
def test_sgemm_is_true_float32(m, n, k):
    g = torch.Generator(device=DEV).manual_seed(4)
    a = torch.randn(m, k, generator=g, device=DEV)
    w = torch.randn(n, k, generator=g, device=DEV)
    out = K().sgemm_nt(a, w)
    ref = (a.double() @ w.double().T)
    # float32 accumulation of k terms: far below what a tensor-core or tf32 mode would leave (1e-3)
    assert float((out.double() - ref).abs().max()) < 1e-5 * math.sqrt(k) * float(ref.abs().max())


def test_sgemm_row_result_does_not_depend_on_the_batch():
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(150, 333, generator=g, device=DEV)
    w = torch.randn(200, 333, generator=g, device=DEV)
    whole = K().sgemm_nt(a, w)
    for i in (0, 63, 64, 149):
        assert torch.equal(whole[i:i + 1], K().sgemm_nt(a[i:i + 1].contiguous(), w))
    assert torch.equal(whole[10:90], K().sgemm_nt(a[10:90].contiguous(), w))


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemv_bf16(m, out_dtype):
    g = torch.Generator(device=DEV).manual_seed(6)
    n, k = 1003, 264 + 1024
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    out = K().gemv_bf16(x, w, out_dtype)
    ref = x.float() @ w.float().T
    assert out.dtype == out_dtype
    if out_dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-4)
    else:
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), **ulp_tol(torch.bfloat16))


@pytest.mark.parametrize("m", [1, 2, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k,split,wide", [(1003, 264, 0, -1), (4096, 4096, 0, -1), (96, 1288, 8, 0), (130, 12288, 3, 1),
                                           (6144, 520, 2, 1), (50, 64, 1, 0), (40, 8, 0, -1), (200, 2048, 6, 0),
                                           (15000, 128, 0, -1)])
def test_gemm_skinny_bf16(m, n, k, split, wide):
    g = torch.Generator(device=DEV).manual_seed(m * 1000 + n)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    ref = x.float() @ w.float().T
    out32 = K().gemm_skinny_bf16(x, w, torch.float32, n_split=split, wide=wide)
    torch.testing.assert_close(out32, ref, rtol=1e-4, atol=2e-4 * math.sqrt(k))
    out16 = K().gemm_skinny_bf16(x, w, torch.bfloat16, n_split=split, wide=wide)
    torch.testing.assert_close(out16.float(), ref.to(torch.bfloat16).float(), **ulp_tol(torch.bfloat16))
    assert torch.equal(out32, K().gemm_skinny_bf16(x, w, torch.float32, n_split=split, wide=wide)), "same bits from run to run"


@pytest.mark.parametrize("inter,k", [(48, 136), (50, 1000), (12288, 4096), (7, 64), (1001, 1288)])
def test_gemv_swiglu_bf16(inter, k):
    g = torch.Generator(device=DEV).manual_seed(k + inter)
    x = torch.randn(1, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g, device=DEV) * (2.0 / math.sqrt(k))).to(torch.bfloat16)
    fused = K().gemv_swiglu_bf16(x, w)
    two_steps = K().swiglu(K().gemv_bf16(x, w, torch.bfloat16))
    assert fused.shape == (1, inter) and torch.equal(fused, two_steps)
    gu = x.float() @ w.float().T
    gate, up = gu[:, :inter].to(torch.bfloat16).float(), gu[:, inter:].to(torch.bfloat16).float()
    torch.testing.assert_close(fused.float(), gate / (1 + torch.exp(-gate)) * up, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m,inter,k,split,wide", [(2, 48, 136, 0, -1), (8, 50, 1000, 2, 0), (5, 132, 4096, 4, 1),
                                                  (8, 12288, 4096, 0, -1), (13, 39, 264, 1, 1), (8, 7, 64, 0, 0)])
def test_gemm_skinny_swiglu_bf16(m, inter, k, split, wide):
    """The gate/up product of decode batches with the SwiGLU in its last step: the skinny product followed by
    the SwiGLU kernel up to the rounding of the sums, and close to a float32 computation of both."""
    g = torch.Generator(device=DEV).manual_seed(m * 7 + k + inter)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g, device=DEV) * (2.0 / math.sqrt(k))).to(torch.bfloat16)
    fused = K().gemm_skinny_swiglu_bf16(x, w, n_split=split, wide=wide)
    two_steps = K().swiglu(K().gemm_skinny_bf16(x, w, torch.bfloat16, n_split=split, wide=wide))
    # the two kernels walk K from different starts (each CTA from its own), so the sums differ in their rounding
    assert fused.shape == (m, inter)
    torch.testing.assert_close(fused.float(), two_steps.float(), rtol=3e-2, atol=3e-2)
    assert torch.equal(fused, K().gemm_skinny_swiglu_bf16(x, w, n_split=split, wide=wide)), "same bits from run to run"
    gu = x.float() @ w.float().T
    gate, up = gu[:, :inter].to(torch.bfloat16).float(), gu[:, inter:].to(torch.bfloat16).float()
    torch.testing.assert_close(fused.float(), gate / (1 + torch.exp(-gate)) * up, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (8, 100, 1000), (5, 264, 4096), (16, 4096, 4096), (8, 24576, 512), (3, 777, 72),
                                   (8, 4096, 12288), (2, 151936, 256), (13, 6144, 4096), (17, 264, 4096), (32, 4096, 4096),
                                   (33, 777, 72), (64, 6144, 4096), (48, 24576, 512), (64, 19456, 1024), (20, 19456, 512),
                                   (64, 4096, 12288)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_streamk_bf16(m, n, k, out_dtype):
    """The decode product that cuts W evenly over the SMs: tiles whose parts lie in several CTAs are summed in
    one order (same bits from run to run), and the flags are clear again after every call."""
    g = torch.Generator(device=DEV).manual_seed(m * 1000 + n + k)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    flag = K().tcgen05_error_flag(x.device)
    flag.zero_()
    out = K().gemm_streamk_bf16(x, w, out_dtype)
    again = K().gemm_streamk_bf16(x, w, out_dtype)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait of the kernel ran out"
    ref = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(k))
    else:
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), **ulp_tol(torch.bfloat16))
    assert torch.equal(out, again), "same bits from run to run"
    from garlic_inference_b200.ops.kernels import _streamk_workspace
    assert int(_streamk_workspace(x.device)[1].abs().sum().item()) == 0, "a flag was left set"


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_call_works(gpu_models):
    """The stream-K product with the flags that announce partial sums held back (a switch of the kernel for this
    test): the CTAs that hold the head of a cut tile poll 2,000 times for a flag that nothing sets, give up, record
    code 34 and return.  The kernel ends (no hang), `Engine.check()` raises, the flag and the hand-over flags are
    clean afterwards, and the same product then gives the right result."""
    from garlic_inference_b200.ops.kernels import WaitRanOut, _streamk_workspace
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn(8, 4096, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(4096, 4096, generator=g, device=DEV) * 0.1).to(torch.bfloat16)     # 32 tiles over 148 CTAs: every tile is cut
    ref = x.float() @ w.float().T
    flag = K().tcgen05_error_flag(x.device)
    flag.zero_()
    model = gpu_models("A", "bfloat16")
    model.engine.check()                                  # nothing pending
    K().streamk_test_unanswered_flags(2000)
    try:
        K().gemm_streamk_bf16(x, w, torch.float32)
        torch.cuda.synchronize()                          # comes back: the wait was bounded
    finally:
        K().streamk_test_unanswered_flags(0)
    assert int(flag.item()) == 34
    with pytest.raises(WaitRanOut, match="code 34"):
        model.engine.check()
    assert int(flag.item()) == 0 and int(_streamk_workspace(x.device)[1].abs().sum().item()) == 0
    model.engine.check()                                  # reported once
    out = K().gemm_streamk_bf16(x, w, torch.float32)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(4096))
    # flags that a kernel which gave up left set (announced, never answered) are cleared by the check as well
    _streamk_workspace(x.device)[1][3] = 1
    flag.fill_(33)
    with pytest.raises(WaitRanOut, match="code 33"):
        K().check_bounded_waits(x.device)
    assert int(_streamk_workspace(x.device)[1].abs().sum().item()) == 0
    out = K().gemm_streamk_bf16(x, w, torch.float32)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(4096))


@pytest.mark.parametrize("m,inter,k", [(300, 128, 64), (300, 100, 64), (257, 7, 128), (2048, 320, 256), (513, 1000, 4096), (129, 136, 72), (1, 264, 1288),
                                       (1024, 12288, 512)])
def test_gemm_tcgen05_swiglu_bf16(m, inter, k):
    """The gate/up product with the SwiGLU in its epilogue: the bits of the plain tcgen05 product followed by
    the SwiGLU kernel, and close to a float32 computation of both."""
    g = torch.Generator(device=DEV).manual_seed(m + inter + k)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, generator=g, device=DEV) * (2.0 / math.sqrt(k))).to(torch.bfloat16)
    flag = K().tcgen05_error_flag(x.device)
    flag.zero_()
    fused = K().gemm_tcgen05_swiglu_bf16(x, w)
    two_steps = K().swiglu(K().gemm_tcgen05_bf16(x, w, torch.bfloat16))
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait of the kernel ran out"
    assert fused.shape == (m, inter) and torch.equal(fused, two_steps)
    gu = x.float() @ w.float().T
    gate, up = gu[:, :inter].to(torch.bfloat16).float(), gu[:, inter:].to(torch.bfloat16).float()
    ref = gate / (1 + torch.exp(-gate)) * up
    torch.testing.assert_close(fused.float(), ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (2048, 512, 256), (300, 1000, 4096), (1, 264, 72), (129, 257 * 8, 1288),
                                   (2048, 6144, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_bf16(m, n, k, out_dtype):
    g = torch.Generator(device=DEV).manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g, device=DEV) * 0.1).to(torch.bfloat16)
    flag = K().tcgen05_error_flag(x.device)
    flag.zero_()
    out = K().gemm_tcgen05_bf16(x, w, out_dtype)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait of the kernel ran out"
    ref = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-4, atol=2e-4 * math.sqrt(k))
    else:
        torch.testing.assert_close(out.float(), ref.to(torch.bfloat16).float(), **ulp_tol(torch.bfloat16))


def test_kernels_refuse_what_they_cannot_take():
    from garlic_inference_b200.ops import KernelError
    x = torch.zeros(9, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(32, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="1 to 8"):
        K().gemv_bf16(x, w, torch.float32)
    with pytest.raises(KernelError, match="multiple of 8"):
        K().gemv_bf16(x[:2, :60].contiguous(), w[:, :60].contiguous(), torch.float32)
    with pytest.raises(KernelError, match="not dense"):
        K().swiglu(x[:, ::2])
    with pytest.raises(KernelError, match="GPU only"):
        K().swiglu(x.cpu())
    q = torch.zeros(2, 4, 20, dtype=torch.float32, device=DEV)
    pool = torch.zeros(4, 2, 16, 20, dtype=torch.float32, device=DEV)
    bt = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="multiple of 8"):
        K().attention_generic(q, pool, pool, bt, z, z, 1.0, 0, z[:1])


# ------------------------------------------------------------------ cache write + attention
def make_cache(n_seqs, lens, n_kv, d, page_size, dtype, seed, spare_pages=3):
    """Pools filled with random keys and values for sequences of the given lengths, pages handed out
    in a shuffled order; returns (k_pool, v_pool, block_table, k_dense, v_dense) with the dense copies
    [seq][len, n_kv, d] in float32."""
    rng = np.random.default_rng(seed)
    g = torch.Generator(device=DEV).manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lens]
    n_pages = sum(pages_per) + spare_pages
    order = rng.permutation(n_pages).tolist()
    max_pages = max(pages_per) + 1
    bt = torch.full((n_seqs, max_pages), -1, dtype=torch.int32)
    k_pool = torch.zeros(n_pages, n_kv, page_size, d, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    k_dense, v_dense = [], []
    for s, n in enumerate(lens):
        k = torch.randn(n, n_kv, d, generator=g, device=DEV).to(dtype)
        v = torch.randn(n, n_kv, d, generator=g, device=DEV).to(dtype)
        for lp in range(pages_per[s]):
            page = order.pop()
            bt[s, lp] = page
            lo, hi = lp * page_size, min(n, (lp + 1) * page_size)
            k_pool[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_pool[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        k_dense.append(k.float()), v_dense.append(v.float())
    return k_pool, v_pool, bt.to(DEV), k_dense, v_dense


def ref_attention(q, k, v, pos, scale, window):
    """One token: q [n_q, d] against keys [len, n_kv, d] up to `pos`, in float64."""
    n_q, n_kv = q.shape[0], k.shape[1]
    lo = max(0, pos - window + 1) if window else 0
    out = torch.empty_like(q, dtype=torch.float64)
    for h in range(n_q):
        kh, vh = k[lo:pos + 1, h // (n_q // n_kv)].double(), v[lo:pos + 1, h // (n_q // n_kv)].double()
        out[h] = torch.softmax(kh @ q[h].double() * scale, 0) @ vh
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,page,window", [
    (4, 4, 16, 16, 0), (5, 1, 48, 8, 0), (6, 1, 32, 16, 20), (8, 2, 128, 32, 0), (2, 1, 256, 16, 33),
    (10, 2, 80, 64, 0)])
def test_attention_generic(dtype, n_q, n_kv, d, page, window):
    lens = [1, 37, 130, page, page + 1]
    k_pool, v_pool, bt, kd, vd = make_cache(len(lens), lens, n_kv, d, page, dtype, seed=d + n_q)
    # tokens: for each sequence its last position, plus some earlier ones (prefill-like rows)
    toks = [(s, n - 1) for s, n in enumerate(lens)] + [(2, 0), (2, 31), (2, 32), (2, 63), (2, 64), (1, 19), (-1, 0)]
    g = torch.Generator(device=DEV).manual_seed(7)
    q = torch.randn(len(toks), n_q, d, generator=g, device=DEV).to(dtype)
    slot = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 0.37
    out = K().attention_generic(q, k_pool, v_pool, bt, pos, slot, scale, window, status).float().view(len(toks), n_q, d)
    assert int(status.item()) == 0
    for i, (s, p) in enumerate(toks):
        if s < 0:
            assert float(out[i].abs().sum()) == 0, "a padding row gives zeros"
            continue
        ref = ref_attention(q[i].float(), kd[s], vd[s], p, scale, window).float()
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(out[i], ref, **tol, msg=lambda m: f"token {i} (seq {s}, pos {p}): {m}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Scores are made so that one key far back takes all the weight: the output must be its value.
    A kernel that drops a chunk, a page or the first or last key fails here, not in the noise."""
    n_q, n_kv, d, page = 4, 2, 64, 16
    n = 700
    for far in (0, 1, 15, 16, 31, 32, 333, 698, 699):
        k_pool, v_pool, bt, kd, vd = make_cache(1, [n], n_kv, d, page, dtype, seed=far)
        q = torch.zeros(1, n_q, d, device=DEV)
        for h in range(n_q):
            q[0, h] = kd[0][far, h // 2] * 4.0          # aligned with key `far`: score ~ 4 |k|^2 against ~ N(0, 4|k|)
        q = q.to(dtype)
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = K().attention_generic(q, k_pool, v_pool, bt, torch.tensor([n - 1], dtype=torch.int32, device=DEV), z,
                                    1.0, 0, z.clone()).float().view(n_q, d)
        for h in range(n_q):
            torch.testing.assert_close(out[h], vd[0][far, h // 2], rtol=2e-2, atol=2e-2,
                                       msg=lambda m: f"far key {far}, head {h}: {m}")
        # with a window that ends just short of it the far key must be gone
        if far < n - 40:
            out_w = K().attention_generic(q, k_pool, v_pool, bt, torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                          z, 1.0, n - 1 - far, z.clone()).float().view(n_q, d)
            assert float((out_w[0] - vd[0][far, 0]).abs().max()) > 0.1
            out_in = K().attention_generic(q, k_pool, v_pool, bt, torch.tensor([n - 1], dtype=torch.int32, device=DEV),
                                           z, 1.0, n - far, z.clone()).float().view(n_q, d)
            torch.testing.assert_close(out_in[0], vd[0][far, 0], rtol=2e-2, atol=2e-2)


def test_attention_generic_same_bits_in_any_batch_and_any_pages():
    n_q, n_kv, d, page = 6, 2, 32, 16
    lens = [90, 300]
    a = make_cache(2, lens, n_kv, d, page, torch.float32, seed=1)
    b = make_cache(2, lens, n_kv, d, page, torch.float32, seed=1, spare_pages=9)     # same numbers, other pages
    g = torch.Generator(device=DEV).manual_seed(8)
    q = torch.randn(5, n_q, d, generator=g, device=DEV)
    slot = torch.tensor([0, 1, 1, 0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([89, 299, 17, 40, 128], dtype=torch.int32, device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    whole = K().attention_generic(q, a[0], a[1], a[2], pos, slot, 0.2, 0, st)
    other = K().attention_generic(q, b[0], b[1], b[2], pos, slot, 0.2, 0, st)
    assert torch.equal(whole, other), "where the pages lie must not matter"
    for i in range(5):
        one = K().attention_generic(q[i:i + 1].contiguous(), a[0], a[1], a[2], pos[i:i + 1].contiguous(),
                                    slot[i:i + 1].contiguous(), 0.2, 0, st)
        assert torch.equal(whole[i:i + 1], one), "a token's result must not depend on the batch"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d,rot,qk_norm,wdt", [
    (4, 2, 16, 16, True, torch.bfloat16), (6, 1, 32, 32, True, torch.float32), (5, 5, 48, 48, True, torch.float32),
    (3, 1, 64, 32, True, torch.float32), (2, 2, 128, 128, False, torch.float32), (2, 1, 80, 0, False, torch.float32),
    (4, 2, 64, 64, True, torch.bfloat16), (8, 2, 128, 128, True, torch.bfloat16), (2, 1, 192, 192, True, torch.float32),
    (2, 2, 256, 256, True, torch.float32)])
def test_qk_norm_rope_append(dtype, n_q, n_kv, d, rot, qk_norm, wdt):
    import plain_qwen3 as plain
    from garlic_inference_b200.parts.rotary import RotaryPositions
    page, n_pages, max_pages, max_pos, theta, eps = 8, 12, 6, 48, 1e4, 1e-5
    g = torch.Generator(device=DEV).manual_seed(d)
    toks = [(0, 0), (0, 1), (0, 7), (0, 8), (1, 30), (-1, 3), (1, 31), (1, 32)]
    n = len(toks)
    qkv = torch.randn(n, (n_q + 2 * n_kv) * d, generator=g, device=DEV).to(dtype)
    qw = (1 + 0.2 * torch.randn(d, generator=g, device=DEV)).to(wdt) if qk_norm else None
    kw = (1 + 0.2 * torch.randn(d, generator=g, device=DEV)).to(wdt) if qk_norm else None
    if rot:
        cos, sin = (t.to(DEV) for t in RotaryPositions.build_tables(rot, theta, max_pos))
    else:
        cos = sin = torch.zeros(max_pos, 0, device=DEV)
    bt = torch.tensor([[3, 9, -1, -1, -1, -1], [0, 1, 2, 11, 5, -1]], dtype=torch.int32, device=DEV)
    k_pool = torch.zeros(n_pages, n_kv, page, d, dtype=dtype, device=DEV)
    v_pool = torch.zeros_like(k_pool)
    slot = torch.tensor([s for s, _ in toks], dtype=torch.int32, device=DEV)
    pos = torch.tensor([p for _, p in toks], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_out = K().qk_norm_rope_append(qkv, n_q, n_kv, d, qw, kw, eps, cos, sin, rot, pos, slot, k_pool, v_pool, bt, status)
    assert int(status.item()) == 0

    x = qkv.float().cpu()
    q_ref = x[:, :n_q * d].view(n, n_q, d)
    k_ref = x[:, n_q * d:(n_q + n_kv) * d].view(n, n_kv, d)
    v_ref = x[:, (n_q + n_kv) * d:].view(n, n_kv, d)
    if qk_norm:
        q_ref = plain.rms_norm(q_ref, qw.float().cpu(), eps)
        k_ref = plain.rms_norm(k_ref, kw.float().cpu(), eps)
    if rot:
        pcpu = pos.cpu()
        q_ref = torch.cat([plain.apply_rope(q_ref[..., :rot], pcpu, theta), q_ref[..., rot:]], -1)
        k_ref = torch.cat([plain.apply_rope(k_ref[..., :rot], pcpu, theta), k_ref[..., rot:]], -1)
    tol = ulp_tol(dtype) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(q_out.float().cpu(), q_ref.to(dtype).float(), **tol)
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for i, (s, p) in enumerate(toks):
        if s < 0:
            continue
        pg, off = int(bt[s, p // page]), p % page
        written[pg, off] = True
        torch.testing.assert_close(k_pool[pg, :, off].float().cpu(), k_ref[i].to(dtype).float(), **tol)
        assert torch.equal(v_pool[pg, :, off].cpu(), v_ref[i].to(dtype)), "values are copied as they are"
    untouched = ~written.view(n_pages, 1, page, 1).expand(-1, n_kv, -1, d)
    assert float(k_pool.float().cpu()[untouched].abs().sum()) == 0 and float(v_pool.float().cpu()[untouched].abs().sum()) == 0

    # a reader of another layer's cache: q as before, nothing written
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    q2 = K().qk_norm_rope_append(qkv, n_q, n_kv, d, qw, kw, eps, cos, sin, rot, pos, slot, k2, v2, bt, status, append=False)
    assert torch.equal(q2, q_out) and float(k2.float().abs().sum()) == 0 and float(v2.float().abs().sum()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_q,n_kv,d", [(5, 1, 64), (8, 2, 128), (3, 3, 192), (1, 1, 256)])
def test_qk_norm_rope_append_of_a_prompt_equals_token_by_token(dtype, n_q, n_kv, d):
    """From 256 tokens on a warp takes four heads of a token at a time (groups that hold query, key and
    value heads at once when the head counts are no multiples of four): the same bits as the same tokens
    in small steps, which the test above compares with the plain implementation."""
    from garlic_inference_b200.parts.rotary import RotaryPositions
    page, n, max_pos = 16, 300, 320
    g = torch.Generator(device=DEV).manual_seed(n_q * 100 + d)
    qkv = torch.randn(n, (n_q + 2 * n_kv) * d, generator=g, device=DEV).to(dtype)
    qw = (1 + 0.2 * torch.randn(d, generator=g, device=DEV)).to(torch.bfloat16)
    kw = (1 + 0.2 * torch.randn(d, generator=g, device=DEV)).to(torch.bfloat16)
    cos, sin = (t.to(DEV) for t in RotaryPositions.build_tables(d, 1e4, max_pos))
    n_pages = max_pos // page
    bt = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32).view(1, -1).to(DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    slot = torch.zeros(n, dtype=torch.int32, device=DEV)
    slot[17] = slot[299] = -1                                   # padding rows: q written, nothing cached
    status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def run(cuts):
        k_pool = torch.zeros(n_pages, n_kv, page, d, dtype=dtype, device=DEV)
        v_pool = torch.zeros_like(k_pool)
        outs = [K().qk_norm_rope_append(qkv[a:b].contiguous(), n_q, n_kv, d, qw, kw, 1e-6, cos, sin, d,
                                        pos[a:b].contiguous(), slot[a:b].contiguous(), k_pool, v_pool, bt, status)
                for a, b in cuts]
        return torch.cat(outs), k_pool, v_pool

    whole = run([(0, n)])
    pieces = run([(a, min(a + 100, n)) for a in range(0, n, 100)])
    assert int(status.item()) == 0
    for a, b in zip(whole, pieces):
        assert torch.equal(a, b)
    assert float(whole[1][bt[0, 1].item(), :, 1].float().abs().sum()) == 0      # position 17: padding


def test_out_of_range_indices_set_the_status_and_touch_nothing():
    n_q, n_kv, d, page = 2, 1, 16, 8
    qkv = torch.ones(2, (n_q + 2) * d, device=DEV)
    cos = sin = torch.zeros(16, d // 2, device=DEV)
    bt = torch.tensor([[0, -1]], dtype=torch.int32, device=DEV)
    pool = torch.zeros(2, n_kv, page, d, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    slot = torch.zeros(2, dtype=torch.int32, device=DEV)
    pos = torch.tensor([3, 9], dtype=torch.int32, device=DEV)           # position 9 lies on an unmapped page
    K().qk_norm_rope_append(qkv, n_q, n_kv, d, None, None, 1e-6, cos, sin, d, pos, slot, pool, pool.clone(), bt, status)
    assert int(status.item()) == 2
    assert float(pool[1].abs().sum()) == 0


# ------------------------------------------------------------------ sampling
def test_greedy_takes_the_lowest_of_equal_maxima():
    logits = torch.full((4, 5003), -1.0, device=DEV)
    logits[0, [4000, 77, 5002]] = 3.0
    logits[1, 5002] = 9.0
    logits[2, 0] = 0.5
    logits[3] = float("-inf")
    out = K().sample(logits, None, None, None, 0)
    assert out.tolist() == [77, 5002, 0, 0]
    view = torch.zeros(3, 100, device=DEV)
    view[:, 7] = 1.0
    assert K().sample(view[:, :50], None, None, None, 0).tolist() == [7, 7, 7]      # rows with a stride


def test_temperature_draws_follow_the_softmax_and_the_key():
    vocab, n = 11, 20000
    g = torch.Generator(device=DEV).manual_seed(9)
    row = torch.randn(vocab, generator=g, device=DEV) * 2
    logits = row.expand(n, vocab).contiguous()
    temps = torch.full((n,), 0.7, device=DEV)
    streams = torch.arange(n, dtype=torch.int64, device=DEV)
    counters = torch.zeros(n, dtype=torch.int32, device=DEV)
    draws = K().sample(logits, temps, streams, counters, 1234)
    freq = torch.bincount(draws.long(), minlength=vocab).float().cpu() / n
    p = torch.softmax(row.cpu() / 0.7, 0)
    assert float((freq - p).abs().max()) < 4 * math.sqrt(0.25 / n) + 1e-3
    assert torch.equal(draws, K().sample(logits, temps, streams, counters, 1234)), "same key, same draw"
    assert not torch.equal(draws, K().sample(logits, temps, streams, counters, 1235))
    # a row's draw depends on its key (seed, stream, counter) only, not on its place in the batch
    perm = torch.randperm(n, device=DEV)
    again = K().sample(logits, temps, streams[perm].contiguous(), counters, 1234)
    assert torch.equal(again, draws[perm])
    # the kernel's generator is the documented one
    from garlic_inference_b200.ops import lib
    u = lib().gi_sample_uniform(1234, 5, 0, 3)
    z = logits[5].cpu() / 0.7 - torch.log(-torch.log(torch.tensor(
        [lib().gi_sample_uniform(1234, 5, 0, i) for i in range(vocab)])))
    assert 0.0 < u < 1.0 and int(z.argmax()) == int(draws[5])
    # temperature 0 in a mixed batch is greedy
    temps[:10] = 0.0
    mixed = K().sample(logits, temps, streams, counters, 1234)
    assert mixed[:10].tolist() == [int(row.argmax())] * 10 and torch.equal(mixed[10:], draws[10:])


def test_a_token_that_cannot_be_drawn_is_never_drawn_at_a_real_vocabulary():
    """A uniform of exactly 1 would give an infinite Gumbel term and let any entry win whatever its logit
    (one in 2^24 per entry with a 24-bit uniform: about 1 % of the draws at 151,936 entries).  Every entry
    but five is at -1e30 here; over 4,096 rows of the full vocabulary none of them may be drawn."""
    vocab, n = 151936, 4096
    logits = torch.full((n, vocab), -1e30, device=DEV)
    allowed = torch.tensor([3, 70000, 100001, 151000, 151935], device=DEV)
    logits[:, allowed] = torch.tensor([0.0, 0.3, -0.2, 0.1, 0.0], device=DEV)
    temps = torch.full((n,), 1.5, device=DEV)
    streams = torch.arange(n, dtype=torch.int64, device=DEV)
    for counter in range(3):
        counters = torch.full((n,), counter, dtype=torch.int32, device=DEV)
        draws = K().sample(logits, temps, streams, counters, 77)
        assert bool(torch.isin(draws.long(), allowed).all()), "a token at -1e30 was drawn"
    freq = torch.bincount(draws.long(), minlength=vocab)[allowed].float().cpu() / n
    p = torch.softmax(torch.tensor([0.0, 0.3, -0.2, 0.1, 0.0]) / 1.5, 0)
    assert float((freq - p).abs().max()) < 4 * math.sqrt(0.25 / n)


# ------------------------------------------------------------------ random weights
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_random_normal_kernel_gives_the_host_generator_s_bits(dtype):
    from garlic_inference_b200.weights.random_init import normal_values, tensor_key
    for name, n, mean, std in [("model.embed_tokens.weight", 100003, 0.0, 0.02), ("model.norm.weight", 96, 1.0, 0.2),
                               ("x", 1, 0.0, 1.0), ("model.layers.3.mlp.up_proj.weight", 1 << 20, 0.0, 0.05)]:
        key = tensor_key(11, name)
        got = K().random_normal(torch.empty(n, dtype=dtype, device=DEV), key, mean, std).cpu()
        want = torch.from_numpy(normal_values(key, n, mean, std)).to(dtype)
        assert torch.equal(got, want), (name, dtype)
    big = K().random_normal(torch.empty(1 << 22, dtype=torch.float32, device=DEV), 5, 0.0, 1.0)
    assert abs(float(big.mean())) < 3e-3 and abs(float(big.std()) - 1.0) < 3e-3


def test_a_folder_written_on_the_cpu_and_a_model_made_on_the_gpu_hold_the_same_tensors(tmp_path):
    import tiny
    from garlic_inference_b200 import AutoModel, write_random_model
    from garlic_inference_b200.weights import Checkpoint
    cfg = tiny.make_config("B")
    folder = write_random_model(tmp_path / "m", cfg, seed=21, std=0.05, norm_std=0.2)
    on_gpu = write_random_model(tmp_path / "g", cfg, seed=21, std=0.05, norm_std=0.2, device="cuda")
    assert (folder / "model.safetensors").read_bytes() == (on_gpu / "model.safetensors").read_bytes()
    model = AutoModel.from_random(cfg, seed=21, device=0, dtype="bfloat16", std=0.05, norm_std=0.2, max_tokens=256,
                                  page_size=16)
    ck = Checkpoint(folder)
    mixer = model.model.blocks[2].mixer
    q_rows = mixer.n_q * mixer.d
    assert torch.equal(mixer.w_qkv[:q_rows].cpu(), ck.tensor("model.layers.2.self_attn.q_proj.weight"))
    assert torch.equal(mixer.w_o.cpu(), ck.tensor("model.layers.2.self_attn.o_proj.weight"))
    assert torch.equal(mixer.k_norm.cpu(), ck.tensor("model.layers.2.self_attn.k_norm.weight"))
    assert torch.equal(model.model.head.weight.cpu(), ck.tensor("lm_head.weight"))


# ------------------------------------------------------------------ tensor-core attention (bfloat16)
def _tiles_for(runs):
    """runs: (slot, first row, rows, first position) per sequence -> int32 [n, 4] cut at 64 rows."""
    out = []
    for slot, row0, n, pos0 in runs:
        for r0 in range(0, n, 64):
            out.append((slot, row0 + r0, min(64, n - r0), pos0 + r0))
    return torch.tensor(out, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("n_q,n_kv,d,page,window", [
    (4, 4, 16, 16, 0), (5, 1, 48, 8, 0), (6, 1, 32, 16, 20), (8, 2, 128, 64, 0), (4, 2, 128, 32, 70),
    (10, 2, 80, 64, 0), (3, 3, 112, 16, 0), (2, 1, 64, 128, 130)])
def test_attention_prefill_bf16(n_q, n_kv, d, page, window):
    lens = [1, 37, 200, 64, 65, 130]
    new = [1, 37, 150, 64, 3, 129]           # the last `new` positions of each sequence are this step's queries
    k_pool, v_pool, bt, kd, vd = make_cache(len(lens), lens, n_kv, d, page, torch.bfloat16, seed=d + n_q)
    runs, row = [], 0
    for s, (n, m) in enumerate(zip(lens, new)):
        runs.append((s, row, m, n - m))
        row += m
    row += 2                                   # two padding rows at the end, in no tile
    g = torch.Generator(device=DEV).manual_seed(17)
    q = torch.randn(row, n_q, d, generator=g, device=DEV).to(torch.bfloat16)
    scale = d ** -0.5
    out = K().attention_prefill_bf16(q, k_pool, v_pool, bt, _tiles_for(runs), scale, window).float().view(row, n_q, d)
    assert float(out[-2:].abs().sum()) == 0
    for s, row0, m, pos0 in runs:
        for i in range(m):
            ref = ref_attention(q[row0 + i].float(), kd[s], vd[s], pos0 + i, scale, window).float()
            torch.testing.assert_close(out[row0 + i], ref, rtol=2e-2, atol=2e-2,
                                       msg=lambda msg: f"seq {s} position {pos0 + i}: {msg}")


@pytest.mark.parametrize("n_q,n_kv,d,page,window,splits", [
    (4, 4, 16, 16, 0, None), (5, 1, 48, 8, 0, 3), (6, 1, 32, 16, 20, None), (32, 8, 128, 64, 0, None),
    (8, 2, 128, 32, 70, 1), (16, 1, 80, 64, 0, 32), (3, 3, 112, 16, 0, 7), (10, 2, 64, 128, 130, 2)])
def test_attention_decode_bf16(n_q, n_kv, d, page, window, splits):
    lens = [1, 37, 700, 64, 65, 130, 63]
    k_pool, v_pool, bt, kd, vd = make_cache(len(lens), lens, n_kv, d, page, torch.bfloat16, seed=d + n_q + 1)
    slots = [0, 1, 2, 3, -1, 4, 5, 6]                                   # one padding row in the middle
    pos = [lens[s] - 1 if s >= 0 else 0 for s in slots]
    g = torch.Generator(device=DEV).manual_seed(18)
    q = torch.randn(len(slots), n_q, d, generator=g, device=DEV).to(torch.bfloat16)
    scale = d ** -0.5
    out = K().attention_decode_bf16(q, k_pool, v_pool, bt, torch.tensor(pos, dtype=torch.int32, device=DEV),
                                    torch.tensor(slots, dtype=torch.int32, device=DEV), scale, window,
                                    n_splits=splits).float().view(len(slots), n_q, d)
    for i, s in enumerate(slots):
        if s < 0:
            assert float(out[i].abs().sum()) == 0, "a padding row gives zeros"
            continue
        ref = ref_attention(q[i].float(), kd[s], vd[s], pos[i], scale, window).float()
        torch.testing.assert_close(out[i], ref, rtol=2e-2, atol=2e-2, msg=lambda msg: f"seq {s}: {msg}")


@pytest.mark.parametrize("n_q,n_kv,page,window,splits", [(4, 4, 64, 0, 1), (8, 2, 64, 0, 3), (5, 1, 128, 0, 2), (16, 1, 64, 0, 4),
                                                         (4, 2, 64, 70, 2), (2, 1, 128, 200, 5), (32, 8, 64, 0, 0),
                                                         (32, 8, 64, 100, 16)])
def test_attention_decode_tcgen05(n_q, n_kv, page, window, splits):
    d = 128
    lens = [1, 37, 300, 64, 65, 130, 513]
    k_pool, v_pool, bt, kd, vd = make_cache(len(lens), lens, n_kv, d, page, torch.bfloat16, seed=page + n_q + 2)
    slots = [0, 1, 2, 3, -1, 4, 5, 6]                                   # one padding row in the middle
    pos = [lens[s] - 1 if s >= 0 else 0 for s in slots]
    g = torch.Generator(device=DEV).manual_seed(21)
    q = torch.randn(len(slots), n_q, d, generator=g, device=DEV).to(torch.bfloat16)
    scale = d ** -0.5
    flag = K().tcgen05_error_flag(q.device)
    flag.zero_()
    out = K().attention_decode_tcgen05(q, k_pool, v_pool, bt, torch.tensor(pos, dtype=torch.int32, device=DEV),
                                       torch.tensor(slots, dtype=torch.int32, device=DEV), scale, window,
                                       n_splits=splits or None).float().view(len(slots), n_q, d)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait of the kernel ran out"
    for i, s in enumerate(slots):
        if s < 0:
            assert float(out[i].abs().sum()) == 0, "a padding row gives zeros"
            continue
        ref = ref_attention(q[i].float(), kd[s], vd[s], pos[i], scale, window).float()
        torch.testing.assert_close(out[i], ref, rtol=2e-2, atol=2e-2, msg=lambda msg: f"seq {s}: {msg}")


def test_attention_decode_tcgen05_finds_one_far_key():
    """One key among 700 carries all the weight, wherever it lies (a page's edge, the first and the last
    position, another slice): the value of that key comes out; a window that ends just short of it loses it."""
    n_q, n_kv, d, page, n = 4, 2, 128, 64, 700
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    for far in (0, 1, 63, 64, 127, 128, 333, 639, 640, 698, 699):
        k_pool, v_pool, bt, kd, vd = make_cache(1, [n], n_kv, d, page, torch.bfloat16, seed=far + 5)
        q = torch.zeros(1, n_q, d, device=DEV)
        for h in range(n_q):
            q[0, h] = kd[0][far, h // 2] * 2.0
        q = q.to(torch.bfloat16)
        for splits in (1, 3):
            out = K().attention_decode_tcgen05(q, k_pool, v_pool, bt, pos, slot, 1.0, 0, n_splits=splits).float().view(n_q, d)
            for h in range(n_q):
                torch.testing.assert_close(out[h], vd[0][far, h // 2], rtol=2e-2, atol=2e-2,
                                           msg=lambda msg: f"far key {far}, head {h}, {splits} slices: {msg}")
        if far < n - 40:
            gone = K().attention_decode_tcgen05(q, k_pool, v_pool, bt, pos, slot, 1.0, n - 1 - far).float().view(n_q, d)
            assert float((gone[0] - vd[0][far, 0]).abs().max()) > 0.1, "the window's edge lets it in"
    assert int(K().tcgen05_error_flag(q.device).item()) == 0


@pytest.mark.parametrize("kernel", ["decode", "prefill"])
def test_tcgen05_attention_over_thousands_of_keys(kernel):
    """4,100 cached keys (65 tiles, 16 slices in the decode kernel): one far key that carries all the weight is
    found wherever it lies, and with ordinary scores the result agrees with the plain softmax."""
    n_q, n_kv, d, page, n = 8, 2, 128, 64, 4100
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    slot = torch.zeros(1, dtype=torch.int32, device=DEV)
    tiles = _tiles128_for([(0, 0, 1, n - 1)])

    def attend(q, k_pool, v_pool, bt, window=0):
        if kernel == "decode":
            return K().attention_decode_tcgen05(q, k_pool, v_pool, bt, pos, slot, 1.0, window).float().view(n_q, d)
        return K().attention_prefill_tcgen05(q, k_pool, v_pool, bt, tiles, 1.0, window).float().view(n_q, d)

    for far in (0, 2047, 2048, 4099):
        k_pool, v_pool, bt, kd, vd = make_cache(1, [n], n_kv, d, page, torch.bfloat16, seed=far + 9)
        q = torch.zeros(1, n_q, d, device=DEV)
        for h in range(n_q):
            q[0, h] = kd[0][far, h // 4] * 2.0
        out = attend(q.to(torch.bfloat16), k_pool, v_pool, bt)
        for h in range(n_q):
            torch.testing.assert_close(out[h], vd[0][far, h // 4], rtol=2e-2, atol=2e-2,
                                       msg=lambda msg: f"{kernel}: far key {far}, head {h}: {msg}")
    g = torch.Generator(device=DEV).manual_seed(3)
    q = (torch.randn(1, n_q, d, generator=g, device=DEV) * 0.3).to(torch.bfloat16)
    for window in (0, 1000):
        out = attend(q, k_pool, v_pool, bt, window)
        ref = ref_attention(q[0].float(), kd[0], vd[0], n - 1, 1.0, window).float()
        torch.testing.assert_close(out, ref, rtol=2e-2, atol=2e-2)
    assert int(K().tcgen05_error_flag(q.device).item()) == 0


def _tiles128_for(runs):
    out = []
    for slot, row0, n, pos0 in runs:
        for r0 in range(0, n, 128):
            out.append((slot, row0 + r0, min(128, n - r0), pos0 + r0))
    return torch.tensor(out, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("n_q,n_kv,page,window", [(4, 4, 64, 0), (8, 2, 64, 0), (5, 1, 128, 0), (4, 2, 64, 70),
                                                  (2, 1, 128, 200), (32, 8, 64, 0)])
def test_attention_prefill_tcgen05(n_q, n_kv, page, window):
    d = 128
    lens = [1, 37, 300, 64, 65, 130, 513]
    new = [1, 37, 250, 64, 3, 129, 513]        # the last `new` positions of each sequence are this step's queries
    k_pool, v_pool, bt, kd, vd = make_cache(len(lens), lens, n_kv, d, page, torch.bfloat16, seed=page + n_q)
    runs, row = [], 0
    for s, (n, m) in enumerate(zip(lens, new)):
        runs.append((s, row, m, n - m))
        row += m
    row += 2                                   # two padding rows at the end, in no tile
    g = torch.Generator(device=DEV).manual_seed(19)
    q = torch.randn(row, n_q, d, generator=g, device=DEV).to(torch.bfloat16)
    scale = d ** -0.5
    flag = K().tcgen05_error_flag(q.device)
    flag.zero_()
    out = K().attention_prefill_tcgen05(q, k_pool, v_pool, bt, _tiles128_for(runs), scale, window).float().view(row, n_q, d)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0, "a bounded wait of the kernel ran out"
    assert float(out[-2:].abs().sum()) == 0
    for s, row0, m, pos0 in runs:
        for i in range(0, m, 7 if m > 100 else 1):
            ref = ref_attention(q[row0 + i].float(), kd[s], vd[s], pos0 + i, scale, window).float()
            torch.testing.assert_close(out[row0 + i], ref, rtol=2e-2, atol=2e-2,
                                       msg=lambda msg: f"seq {s} position {pos0 + i}: {msg}")


def test_attention_prefill_tcgen05_finds_one_far_key():
    n_q, n_kv, d, page, n = 4, 2, 128, 64, 700
    for far in (0, 1, 63, 64, 127, 128, 333, 639, 640, 698, 699):
        k_pool, v_pool, bt, kd, vd = make_cache(1, [n], n_kv, d, page, torch.bfloat16, seed=far + 3)
        q = torch.zeros(1, n_q, d, device=DEV)
        for h in range(n_q):
            q[0, h] = kd[0][far, h // 2] * 2.0
        q = q.to(torch.bfloat16)
        tiles = _tiles128_for([(0, 0, 1, n - 1)])
        out = K().attention_prefill_tcgen05(q, k_pool, v_pool, bt, tiles, 1.0, 0).float().view(n_q, d)
        for h in range(n_q):
            torch.testing.assert_close(out[h], vd[0][far, h // 2], rtol=2e-2, atol=2e-2,
                                       msg=lambda msg: f"far key {far}, head {h}: {msg}")
        if far < n - 40:
            gone = K().attention_prefill_tcgen05(q, k_pool, v_pool, bt, tiles, 1.0, n - 1 - far).float().view(n_q, d)
            assert float((gone[0] - vd[0][far, 0]).abs().max()) > 0.1, "the window's edge lets it in"
    assert int(K().tcgen05_error_flag(q.device).item()) == 0


@pytest.mark.parametrize("kernel", ["decode", "prefill"])
def test_tensor_core_attention_finds_one_far_key(kernel):
    n_q, n_kv, d, page, n = 8, 2, 64, 16, 700
    for far in (0, 1, 15, 16, 63, 64, 333, 639, 640, 698, 699):
        k_pool, v_pool, bt, kd, vd = make_cache(1, [n], n_kv, d, page, torch.bfloat16, seed=far + 1)
        q = torch.zeros(1, n_q, d, device=DEV)
        for h in range(n_q):
            q[0, h] = kd[0][far, h // 4] * 4.0
        q = q.to(torch.bfloat16)
        pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
        z = torch.zeros(1, dtype=torch.int32, device=DEV)

        def run(window):
            if kernel == "decode":
                return K().attention_decode_bf16(q, k_pool, v_pool, bt, pos, z, 1.0, window).float().view(n_q, d)
            return K().attention_prefill_bf16(q, k_pool, v_pool, bt, _tiles_for([(0, 0, 1, n - 1)]), 1.0,
                                              window).float().view(n_q, d)

        out = run(0)
        for h in range(n_q):
            torch.testing.assert_close(out[h], vd[0][far, h // 4], rtol=2e-2, atol=2e-2,
                                       msg=lambda msg: f"{kernel}: far key {far}, head {h}: {msg}")
        if far < n - 40:
            assert float((run(n - 1 - far)[0] - vd[0][far, 0]).abs().max()) > 0.1, "the window's edge lets it in"
            torch.testing.assert_close(run(n - far)[0], vd[0][far, 0], rtol=2e-2, atol=2e-2)


def test_tensor_core_attention_refuses_other_sizes():
    from garlic_inference_b200.ops import KernelError
    q = torch.zeros(1, 34, 64, dtype=torch.bfloat16, device=DEV)
    pool = torch.zeros(2, 2, 16, 64, dtype=torch.bfloat16, device=DEV)
    bt = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="up to 16"):
        K().attention_decode_bf16(q, pool, pool, bt, z, z, 1.0, 0)
    q2 = torch.zeros(1, 2, 256, dtype=torch.bfloat16, device=DEV)
    pool2 = torch.zeros(2, 2, 16, 256, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="multiple of 16 up to 128"):
        K().attention_decode_bf16(q2, pool2, pool2, bt, z, z, 1.0, 0)
    assert not K().mma_attention_takes(torch.bfloat16, 256) and not K().mma_attention_takes(torch.float32, 64)
    assert K().mma_attention_takes(torch.bfloat16, 48)
