"""Numerics of every sm_100a kernel against the plain PyTorch fp32 formulas (needs a B200)."""
import math

import pytest
import torch

from ksa_b200 import ops
from ksa_b200.ops import _lib, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(torch.bfloat16)


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def check(a, b, tol, what=""):
    _lib.check_status()
    assert torch.isfinite(a.float()).all(), f"{what}: non-finite values"
    e = rel_err(a, b)
    assert e < tol, f"{what}: relative error {e:.3e} >= {tol}"


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 1024, 192), (1000, 264, 72),
                                   (2048, 4096, 2048), (130, 136, 520)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    if a_mn and M % 8:
        pytest.skip("an MN-major operand needs its contiguous extent to be a multiple of 8")
    A = bf(M, K)
    B = bf(N, K)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    c = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    check(c, A.float() @ B.float().t(), 1e-2, f"gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 256), (1000, 264, 72), (2048, 4096, 2048), (8256, 2048, 520)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_cta_pairs(M, N, K, a_mn, b_mn):
    if a_mn and M % 8:
        pytest.skip("an MN-major operand needs its contiguous extent to be a multiple of 8")
    A = bf(M, K)
    B = bf(N, K)
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    c = ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, pair=True)
    check(c, A.float() @ B.float().t(), 1e-2, f"pair gemm {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}")
    out = torch.randn(M, N, device=DEV)
    expect = out + 0.5 * (A.float() @ B.float().t())
    ops.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn, out=out, accumulate=True, alpha=0.5, pair=True)
    check(out, expect, 5e-3, "pair gemm fp32 accumulate")


def test_gemm_fp32_accumulate_and_strided_views():
    M, N, K = 512, 768, 320
    packed = bf(M, 2 * K)
    A = packed[:, K:]                       # row stride 2K
    B = bf(N, K)
    out = torch.randn(M, N, device=DEV)
    expect = out + 0.5 * (A.float() @ B.float().t())
    ops.gemm(A, B, out=out, accumulate=True, alpha=0.5)
    check(out, expect, 5e-3, "gemm fp32 accumulate")


@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 16])
@pytest.mark.parametrize("N,K", [(2560, 4096), (6144, 2560), (19456, 2560), (264, 9728), (151936, 2560)])
def test_skinny_gemm_for_decoding(M, N, K):
    packed = bf(M, K + 64)
    A = packed[:, 32:32 + K]                # strided view with a 64-byte column offset
    B = bf(N, K, scale=0.05)
    out = torch.empty(M, N + 8, device=DEV, dtype=torch.bfloat16)[:, :N]
    before = _lib.launch_count()
    c = ops.gemm(A, B, out=out)
    assert _lib.launch_count() == before + 1
    check(c, A.float() @ B.float().t(), 1e-2, f"skinny gemm {M}x{N}x{K}")


@pytest.mark.parametrize("M", [1, 2, 4, 7, 16])
@pytest.mark.parametrize("F,K", [(1280, 2560), (9728, 2560), (136, 4096)])
def test_skinny_gate_up_projection_with_swiglu(M, F, K):
    """The decode step's gate/up projection applies SwiGLU itself: one launch, equal to projection + activation
    (gate and up rounded to bf16 in between, as the two separate kernels do)."""
    x = bf(M, K)
    w13 = bf(2 * F, K, scale=0.05)
    before = _lib.launch_count()
    with torch.no_grad():
        h = ops.linear_swiglu(x, w13)
    assert _lib.launch_count() == before + 1 and h.shape == (M, F)
    gu = (x.float() @ w13.float().t()).bfloat16().float()
    expect = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    check(h, expect, 1.5e-2, f"gemv swiglu {M}x{2 * F}x{K}")
    # a chain of dependent-launched kernels on one stream: each reads the previous one's output
    w2 = bf(K, F, scale=0.002)     # small enough that the chain does not grow
    with torch.no_grad():
        y = x
        for _ in range(4):
            y = ops.linear(ops.linear_swiglu(y, w13), w2)
    yr = x.float()
    for _ in range(4):
        gu = (yr @ w13.float().t()).bfloat16().float()
        yr = ((torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]).bfloat16().float() @ w2.float().t()).bfloat16().float()
    check(y, yr, 5e-2, "dependent-launch chain")


@pytest.mark.parametrize("M,delta_rows", [(1, 1), (3, 3), (4, 2), (2, 0)])
@pytest.mark.parametrize("glu", [False, True])
def test_skinny_projection_with_residual_add_and_norm(M, delta_rows, glu):
    """The decode step's `x + delta -> RMSNorm -> projection` in one launch against the separate kernels."""
    K, N = 2560, 6144 if not glu else 2 * 1280
    x = bf(M, K)
    delta = bf(delta_rows, K) if delta_rows else None
    nw = (1 + 0.1 * torch.randn(K, device=DEV)).bfloat16()
    w = bf(N, K, scale=0.05)
    before = _lib.launch_count()
    with torch.no_grad():
        res, y = ops.norm_linear(x, delta, nw, 1e-6, w, glu=glu)
        assert _lib.launch_count() == before + 1
        res_ref, h = ops.add_rms_norm(x, delta, nw, 1e-6)
        y_ref = ops.linear_swiglu(h, w) if glu else ops.linear(h, w)
    assert torch.equal(res, res_ref)
    check(y, y_ref.float(), 1.5e-2, f"norm + projection {M}x{N}x{K} glu={glu}")


def test_linear_autograd():
    x = bf(3, 200, 256).requires_grad_()
    w = bf(384, 256, scale=0.05).requires_grad_()
    y = ops.linear(x, w)
    g = bf(3, 200, 384)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    yr = ref.linear(xr, wr)
    yr.backward(g.float())
    check(y, yr, 1e-2, "linear fwd")
    check(x.grad, xr.grad, 1e-2, "linear dx")
    check(w.grad, wr.grad, 1e-2, "linear dw")


def test_linear_main_grad_accumulates_in_fp32():
    x = bf(256, 128)
    w = bf(256, 128, scale=0.05).requires_grad_()
    w.main_grad = torch.zeros(256, 128, device=DEV)
    g = bf(256, 256)
    for _ in range(2):
        ops.linear(x, w).backward(g)
    assert w.grad is None
    check(w.main_grad, 2 * (g.float().t() @ x.float()), 1e-2, "main_grad accumulation")


# ------------------------------------------------------------------ norms / rope / mlp
@pytest.mark.parametrize("rows,D", [(7, 256), (300, 2048), (1500, 2560)])
def test_add_rms_norm(rows, D):
    x, d = bf(rows, D), bf(rows, D)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16)
    xs = [t.clone().requires_grad_() for t in (x, d, w)]
    res, y = ops.add_rms_norm(*xs, 1e-6)
    gr, gy = bf(rows, D), bf(rows, D)
    torch.autograd.backward([res, y], [gr, gy])
    fs = [t.detach().float().requires_grad_() for t in (x, d, w)]
    r_ref = fs[0] + fs[1]
    y_ref = ref.rms_norm(r_ref, fs[2])
    ((r_ref * gr.float()).sum() + (y_ref * gy.float()).sum()).backward()
    check(res, r_ref, 5e-3, "residual")
    check(y, y_ref, 1e-2, "rmsnorm y")
    check(xs[0].grad, fs[0].grad, 1.5e-2, "rmsnorm dx")
    check(xs[2].grad, fs[2].grad, 2e-2, "rmsnorm dw")


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 16, 8), (64, 4, 2)])
@pytest.mark.parametrize("interleaved", [False, True])
def test_qk_norm_rope(D, Hq, Hkv, interleaved):
    T = 333
    qkv = bf(T, (Hq + 2 * Hkv) * D).requires_grad_()
    qw = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    kw = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    pos = torch.randint(0, 100000, (T,), device=DEV)
    out = ops.qk_norm_rope_packed(qkv, qw, kw, pos, Hq, Hkv, D, 1e6, 1e-6, interleaved)
    g = bf(T, (Hq + 2 * Hkv) * D)
    out.backward(g)
    f = [t.detach().float().requires_grad_() for t in (qkv, qw, kw)]
    q = f[0][:, :Hq * D].reshape(1, T, Hq, D)
    k = f[0][:, Hq * D:(Hq + Hkv) * D].reshape(1, T, Hkv, D)
    qr, kr = ref.qk_norm_rope(q, k, f[1], f[2], pos, 1e6, 1e-6, interleaved)
    o_ref = torch.cat([qr.reshape(T, -1), kr.reshape(T, -1), f[0][:, (Hq + Hkv) * D:]], 1)
    o_ref.backward(g.float())
    check(out, o_ref, 1e-2, "qknorm_rope fwd")
    check(qkv.grad, f[0].grad, 2e-2, "qknorm_rope dqkv")
    assert torch.equal(qkv.grad[:, (Hq + Hkv) * D:], g[:, (Hq + Hkv) * D:])
    check(qw.grad, f[1].grad, 3e-2, "q_norm dw")
    check(kw.grad, f[2].grad, 3e-2, "k_norm dw")


def test_swiglu():
    gu = bf(257, 2 * 768).requires_grad_()
    y = ops.swiglu(gu)
    g = bf(257, 768)
    y.backward(g)
    f = gu.detach().float().requires_grad_()
    yr = ref.swiglu(f)
    yr.backward(g.float())
    check(y, yr, 1e-2, "swiglu fwd")
    check(gu.grad, f.grad, 1.5e-2, "swiglu bwd")


def test_embedding():
    table = bf(1000, 256).requires_grad_()
    ids = torch.randint(0, 1000, (4, 77), device=DEV)
    y = ops.embedding(ids, table)
    g = bf(4, 77, 256)
    y.backward(g)
    f = table.detach().float().requires_grad_()
    yr = ref.embedding(ids, f)
    yr.backward(g.float())
    assert torch.equal(y.float(), yr)
    check(table.grad, f.grad, 1e-2, "embedding bwd")


@pytest.mark.parametrize("T,V,chunk", [(300, 4096, 128), (64, 151936, 64)])
def test_linear_cross_entropy(T, V, chunk):
    D = 256
    h = bf(T, D).requires_grad_()
    w = bf(V, D, scale=0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    loss = ops.linear_cross_entropy(h, w, labels, chunk_tokens=chunk)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = ref.linear_cross_entropy(hf, wf, labels)
    lr.backward()
    _lib.check_status()
    assert abs(loss.item() - lr.item()) < 2e-2 * abs(lr.item()), (loss.item(), lr.item())
    check(h.grad, hf.grad, 3e-2, "linear_ce dh")
    check(w.grad, wf.grad, 3e-2, "linear_ce dw")


def test_adamw():
    n = 4096 * 3
    master = torch.randn(n, device=DEV)
    grad = torch.randn(n, device=DEV)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    out = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    sumsq = torch.zeros(1, device=DEV)
    mr, gr_, m_r, v_r = master.clone().cpu(), grad.clone().cpu(), m.clone().cpu(), v.clone().cpu()
    for step in (1, 2, 3):
        hyper = torch.tensor([1e-3, 1 - 0.9 ** step, 1 - 0.95 ** step, 0.5], device=DEV)
        sumsq.zero_()
        ops.adamw_step(master, grad, m, v, out, hyper, 0.9, 0.95, 1e-8, 0.1, clip_value=1.0, sumsq=sumsq)
        sq = ref.adamw_step_(mr, gr_, m_r, v_r, 1e-3, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=0.5, clip_value=1.0)
        assert abs(sumsq.item() - sq.item()) < 1e-3 * sq.item()
    check(master, mr.to(DEV), 1e-5, "adamw master")
    check(out, mr.to(DEV), 5e-3, "adamw bf16 copy")


# ------------------------------------------------------------------ attention
def _attn_inputs(B, L, Hq, Hkv, D, C, S):
    Ns = ((L + C - 1) // C) * S
    mk = lambda T, H: bf(B, T, H, D)
    return [mk(L, Hq), mk(L, Hkv), mk(L, Hkv), mk(Ns, Hq), mk(Ns, Hkv), mk(Ns, Hkv)]


@pytest.mark.parametrize("B,L,Hq,Hkv,D,C,S,W", [
    (1, 1024, 4, 2, 128, 128, 1, 2),
    (2, 2048, 4, 2, 64, 64, 1, 4),
    (1, 1536, 2, 2, 128, 128, 2, 1),      # Hq/Hkv odd -> single slot
    (1, 1280, 8, 2, 128, 8, 1, 16),       # chunk smaller than the tile
    (1, 1000, 4, 2, 128, 128, 1, 3),      # ragged last tile / chunk
])
def test_ksa_attention_fwd_bwd(B, L, Hq, Hkv, D, C, S, W):
    t = _attn_inputs(B, L, Hq, Hkv, D, C, S)
    xs = [x.clone().requires_grad_() for x in t]
    o_t, o_s = ops.ksa_attention(*xs, C, S, W)
    g_t, g_s = bf(*o_t.shape), bf(*o_s.shape)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    fs = [x.detach().float().requires_grad_() for x in t]
    r_t, r_s = ref.ksa_attention(*fs, C, S, W)
    torch.autograd.backward([r_t, r_s], [g_t.float(), g_s.float()])
    check(o_t, r_t, 1.5e-2, "ksa o_text")
    check(o_s, r_s, 1.5e-2, "ksa o_summary")
    names = ["dq_t", "dk_t", "dv_t", "dq_s", "dk_s", "dv_s"]
    for n, a, b_ in zip(names, xs, fs):
        check(a.grad, b_.grad, 3e-2, f"ksa {n}")


@pytest.mark.parametrize("L", [8192, 32768])
def test_ksa_attention_benchmark_shape_against_blockwise_oracle(L):
    """16 query / 8 KV heads of 128, chunk 128 + 1 summary, window 8: forward and backward against the fp32 block-mode
    oracle on the GPU.  At 32768 tokens the 256 summary keys fill two key tiles and every summary key tile's query
    range is split into segments whose fp32 partial sums are folded by the summary-query kernel."""
    B, Hq, Hkv, D, C, S, W = 1, 16, 8, 128, 128, 1, 8
    t = _attn_inputs(B, L, Hq, Hkv, D, C, S)
    xs = [x.clone().requires_grad_() for x in t]
    o_t, o_s = ops.ksa_attention(*xs, C, S, W)
    g_t, g_s = bf(*o_t.shape), bf(*o_s.shape)
    torch.autograd.backward([o_t, o_s], [g_t, g_s])
    fs = [x.detach().float().requires_grad_() for x in t]
    r_t, r_s = ref.ksa_attention_blockwise(*fs, C, S, W, q_block=2048)
    torch.autograd.backward([r_t, r_s], [g_t.float(), g_s.float()])
    check(o_t, r_t, 1.5e-2, "ksa o_text")
    check(o_s, r_s, 1.5e-2, "ksa o_summary")
    for n, a, b_ in zip(["dq_t", "dk_t", "dv_t", "dq_s", "dk_s", "dv_s"], xs, fs):
        check(a.grad, b_.grad, 3e-2, f"ksa {n} L={L}")


def test_attention_backward_deterministic_mode_is_bit_reproducible():
    """With ``ops.set_deterministic(True)`` the text-query backward runs as two kernels that never add across CTAs and
    the summary key tiles are not split: two runs give identical bits, and they match the fused backward to rounding."""
    B, L, Hq, Hkv, D, C, S, W = 1, 2048, 4, 2, 128, 128, 1, 2
    t = _attn_inputs(B, L, Hq, Hkv, D, C, S)
    g_t, g_s = bf(B, L, Hq, D), bf(B, t[3].shape[1], Hq, D)

    def grads():
        xs = [x.clone().requires_grad_() for x in t]
        o_t, o_s = ops.ksa_attention(*xs, C, S, W)
        torch.autograd.backward([o_t, o_s], [g_t, g_s])
        return [x.grad for x in xs]

    fused = grads()
    ops.set_deterministic(True)
    try:
        a, b_ = grads(), grads()
    finally:
        ops.set_deterministic(False)
    for n, x, y, z in zip(["dq_t", "dk_t", "dv_t", "dq_s", "dk_s", "dv_s"], a, b_, fused):
        assert torch.equal(x, y), f"{n} differs between two deterministic runs"
        check(z, x.float(), 2e-2, f"fused vs deterministic {n}")


@pytest.mark.parametrize("L,window", [(1024, -1), (1500, -1), (2048, 300)])
def test_causal_attention_fwd_bwd(L, window):
    B, Hq, Hkv, D = 2, 4, 2, 128
    q, k, v = bf(B, L, Hq, D), bf(B, L, Hkv, D), bf(B, L, Hkv, D)
    xs = [x.clone().requires_grad_() for x in (q, k, v)]
    o = ops.causal_attention(*xs, window=window)
    g = bf(*o.shape)
    o.backward(g)
    fs = [x.detach().float().requires_grad_() for x in (q, k, v)]
    r = ref.causal_attention(*fs, window=window)
    r.backward(g.float())
    check(o, r, 1.5e-2, "causal o")
    for n, a, b_ in zip(["dq", "dk", "dv"], xs, fs):
        check(a.grad, b_.grad, 3e-2, f"causal {n}")


@pytest.mark.parametrize("window", [-1, 200])
@pytest.mark.parametrize("deterministic", [False, True])
def test_causal_attention_over_packed_documents(window, deterministic):
    """``cu_seqlens`` (documents packed into one sequence, boundaries anywhere inside the 128-row tiles): forward and
    backward on the kernels against the dense-mask oracle; no query sees a key of another document."""
    B, L, Hq, Hkv, D = 2, 1500, 4, 2, 128
    cu = torch.tensor([0, 70, 71, 400, 1024, 1300, 1500], device=DEV, dtype=torch.int32)
    q, k, v = bf(B, L, Hq, D), bf(B, L, Hkv, D), bf(B, L, Hkv, D)
    xs = [x.clone().requires_grad_() for x in (q, k, v)]
    ops.set_deterministic(deterministic)
    try:
        o = ops.causal_attention(*xs, window=window, cu_seqlens=cu)
        g = bf(*o.shape)
        o.backward(g)
    finally:
        ops.set_deterministic(False)
    fs = [x.detach().float().requires_grad_() for x in (q, k, v)]
    r = ref.causal_attention(*fs, window=window, cu_seqlens=cu.long())
    r.backward(g.float())
    check(o, r, 1.5e-2, "packed causal o")
    for n, a, b_ in zip(["dq", "dk", "dv"], xs, fs):
        check(a.grad, b_.grad, 3e-2, f"packed causal {n}")
    # a perturbation of document 3's keys leaves the outputs of every other document bit-identical
    k2 = k.clone()
    k2[:, 400:1024] += 1.0
    o2 = ops.causal_attention(q, k2, v, window=window, cu_seqlens=cu)
    assert torch.equal(o2[:, :400], o.detach()[:, :400]) and torch.equal(o2[:, 1024:], o.detach()[:, 1024:])


def test_attention_reads_packed_qkv_views():
    """q/k/v as strided views of one packed projection output (what the model passes)."""
    B, L, Hq, Hkv, D = 1, 512, 4, 2, 128
    packed = bf(B * L, (Hq + 2 * Hkv) * D)
    q = packed[:, :Hq * D].view(B, L, Hq, D)
    k = packed[:, Hq * D:(Hq + Hkv) * D].view(B, L, Hkv, D)
    v = packed[:, (Hq + Hkv) * D:].view(B, L, Hkv, D)
    o = ops.causal_attention(q, k, v)
    r = ref.causal_attention(q.float(), k.float(), v.float())
    check(o, r, 1.5e-2, "packed views")


def test_dual_linear():
    R, n_a, K, N = 520, 400, 256, 384
    x = bf(R, K).requires_grad_()
    wa, wb = bf(N, K, scale=0.05).requires_grad_(), bf(N, K, scale=0.05).requires_grad_()
    y = ops.dual_linear(x, wa, wb, n_a)
    g = bf(R, N)
    y.backward(g)
    xf, waf, wbf = [t.detach().float().requires_grad_() for t in (x, wa, wb)]
    yr = torch.cat([xf[:n_a] @ waf.t(), xf[n_a:] @ wbf.t()])
    yr.backward(g.float())
    check(y, yr, 1e-2, "dual y")
    check(x.grad, xf.grad, 1e-2, "dual dx")
    check(wa.grad, waf.grad, 1e-2, "dual dwa")
    check(wb.grad, wbf.grad, 1e-2, "dual dwb")


def test_add_rms_norm_partial_delta():
    rows, n_d, D = 300, 256, 512
    x, d = bf(rows, D).requires_grad_(), bf(n_d, D).requires_grad_()
    w = (1 + 0.1 * torch.randn(D, device=DEV)).to(torch.bfloat16).requires_grad_()
    res, y = ops.add_rms_norm(x, d, w)
    gr, gy = bf(rows, D), bf(rows, D)
    torch.autograd.backward([res, y], [gr, gy])
    xf, df, wf = [t.detach().float().requires_grad_() for t in (x, d, w)]
    r_ref = xf + torch.cat([df, torch.zeros(rows - n_d, D, device=DEV)])
    y_ref = ref.rms_norm(r_ref, wf)
    ((r_ref * gr.float()).sum() + (y_ref * gy.float()).sum()).backward()
    check(res, r_ref, 5e-3, "partial residual")
    check(y, y_ref, 1e-2, "partial y")
    check(d.grad, df.grad, 1.5e-2, "partial ddelta")
    check(x.grad, xf.grad, 1.5e-2, "partial dx")


@pytest.mark.parametrize("B,L,Hq,Hkv,D,C,S,W", [(2, 1024, 4, 2, 128, 128, 1, 2), (1, 512, 4, 2, 64, 64, 1, 4),
                                                (2, 768, 4, 2, 128, 128, 0, 0)])
def test_attention_packed(B, L, Hq, Hkv, D, C, S, W):
    Ns = (L // C) * S
    R = B * (L + Ns)
    qkv = bf(R, (Hq + 2 * Hkv) * D).requires_grad_()
    kw = dict(chunk=C, n_sum=max(S, 1), window=W) if S > 0 else {}
    out = ops.attention_packed(qkv, B, L, Ns, Hq, Hkv, D, **kw)
    g = bf(R, Hq * D)
    out.backward(g)
    f = qkv.detach().float().cpu().requires_grad_()
    o_ref = ops.attention_packed(f, B, L, Ns, Hq, Hkv, D, **kw)
    o_ref.backward(g.float().cpu())
    check(out, o_ref.to(DEV), 1.5e-2, "packed attention out")
    check(qkv.grad, f.grad.to(DEV), 3e-2, "packed attention dqkv")


# ------------------------------------------------------------------ all-gather -> GEMM in one launch
def _gather_case(world, rank, rows, K):
    """Every rank's copy of a row-sharded [rows_pad, K] buffer as separate tensors of this GPU: a copy holds its own
    shard and junk elsewhere, like the symmetric buffers of a tensor-parallel group before the gather."""
    import ctypes
    shard = (rows + world - 1) // world
    full = bf(shard * world, K)
    copies = []
    for r in range(world):
        c = torch.full_like(full, 7.0)
        c[r * shard:(r + 1) * shard] = full[r * shard:(r + 1) * shard]
        copies.append(c)
    peers = (ctypes.c_void_p * world)(*[c.data_ptr() for c in copies])
    return full, copies, peers, shard


@pytest.mark.parametrize("world,rank,rows,N,K", [(4, 1, 8548, 1536, 512), (2, 0, 4096, 512, 1024),
                                                  (8, 7, 8256, 768, 264), (4, 3, 600, 256, 128)])
def test_all_gather_gemm_one_launch(world, rank, rows, N, K):
    """The math warps read A out of this rank's copy while the communication warps of the same launch fill it from the
    other copies (which here live on the same GPU); two launches in a row check the running completion count."""
    full, copies, peers, shard = _gather_case(world, rank, rows, K)
    W = bf(N, K)
    ready = torch.zeros(world, dtype=torch.int32, device=DEV)
    done = torch.zeros(_lib.GATHER_COUNTERS, dtype=torch.int32, device=DEV)
    want = full[:rows].float() @ W.float().t()
    n_chunks = (shard * K * 2 + 8191) // 8192
    for launch in (1, 2):
        if launch == 2:                       # junk again in the remote shards of the own copy
            keep = copies[rank][rank * shard:(rank + 1) * shard].clone()
            copies[rank].fill_(-3.0)
            copies[rank][rank * shard:(rank + 1) * shard] = keep
        a = copies[rank][:rows]
        out = ops.gemm_gather(a, W, peers, world, rank, shard * K * 2, ready, None, done, dep_operand=1, dep_offset=0)
        check(out, want, 1e-2, f"all-gather gemm launch {launch}")
        assert torch.equal(copies[rank], full), "the gather did not complete the own copy"
        per_shard = done.view(8, 4).sum(1)               # landed chunks per shard: counted afresh by every launch
        expect = torch.zeros(8, dtype=torch.int64, device=DEV)
        expect[:world] = n_chunks
        expect[rank] = 0
        assert torch.equal(per_shard, expect)


def test_gather_rides_along_without_dependency():
    """dep_operand=0: the gather only shares the launch; the GEMM reads unrelated operands."""
    full, copies, peers, shard = _gather_case(4, 2, 4096, 256)
    A, W = bf(1000, 264), bf(520, 264)
    ready = torch.zeros(4, dtype=torch.int32, device=DEV)
    out = ops.gemm_gather(A, W, peers, 4, 2, shard * 256 * 2, ready, None, None, dep_operand=0)
    check(out, A.float() @ W.float().t(), 1e-2, "gemm with a gather riding along")
    assert torch.equal(copies[2], full)


def test_all_gather_gemm_gives_up_when_a_shard_never_becomes_ready():
    """The ready flag of the shards is never raised: the communication CTAs and then the math producers run out of
    their bounded waits, the launch ends with the flag-timeout status, and the next launch works."""
    full, copies, peers, shard = _gather_case(2, 0, 2048, 256)
    W = bf(256, 256)
    ready = torch.zeros(2, dtype=torch.int32, device=DEV)
    done = torch.zeros(_lib.GATHER_COUNTERS, dtype=torch.int32, device=DEV)
    _lib.check_status()
    _lib.set_peer_wait_ms(200)
    try:
        ops.gemm_gather(copies[0][:2048], W, peers, 2, 0, shard * 256 * 2, ready, None, done,
                        dep_operand=1, epoch_add=1)                        # waits for ready[1] >= 1
        with pytest.raises(RuntimeError, match="timed out waiting for a flag"):
            _lib.check_status()
        ready.fill_(1)
        out = ops.gemm_gather(copies[0][:2048], W, peers, 2, 0, shard * 256 * 2, ready, None, done,
                              dep_operand=1, epoch_add=1)
        check(out, full[:2048].float() @ W.float().t(), 1e-2, "all-gather gemm after a timed-out launch")
    finally:
        _lib.set_peer_wait_ms(10000)


@pytest.mark.parametrize("world,M,N,K,shard", [(4, 1000, 512, 264, 260), (2, 4096, 2560, 512, 2048), (8, 8256, 256, 128, 1056),
                                               (4, 1000, 264, 72, 260), (3, 700, 320, 64, 256)])
def test_gemm_scatters_row_blocks_to_their_owners(world, M, N, K, shard):
    """GEMM -> reduce-scatter, producer side: row block r of the product lands in the r-th output buffer (here all
    on one GPU), whatever the alignment of the block boundaries to the 128-row tiles.  With N a multiple of 64 the
    32-row blocks inside one owner's rows leave through TMA stores, the straddling ones and every other N through
    per-row stores."""
    import ctypes
    A, W = bf(M, K), bf(N, K)
    outs = [torch.full((shard, N), 9.0, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[o.data_ptr() for o in outs])
    _lib.call("ksa_gemm2_scatter_bf16", A, W, M, N, K, A.stride(0), W.stride(0), N, ptrs, world, shard)
    want = A.float() @ W.float().t()
    for r in range(world):
        lo, hi = min(r * shard, M), min((r + 1) * shard, M)
        if hi > lo:
            check(outs[r][:hi - lo], want[lo:hi], 1e-2, f"row block {r}")
        assert (outs[r][hi - lo:] == 9.0).all(), "rows beyond the block were written"


# ------------------------------------------------------------------ bounded waits
def test_wait_on_a_flag_nobody_sets_runs_out_and_reports():
    """A device-side wait on a peer flag that nothing ever raises gives up after its limit, leaves a status code that
    the host reads as an exception, and the context stays usable (no trap, no hang)."""
    import time
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    _lib.check_status()
    _lib.set_peer_wait_ms(300)
    try:
        t0 = time.perf_counter()
        _lib.call("ksa_signal_wait", flags, 2, None, 7)          # waits for flags[0..1] >= 7
        with pytest.raises(RuntimeError, match="timed out waiting for a flag"):
            _lib.check_status()
        dt = time.perf_counter() - t0
        assert 0.1 < dt < 5.0, dt
        _lib.check_status()                                      # cleared: the next check is clean
        flags.fill_(7)
        _lib.call("ksa_signal_wait", flags, 2, None, 7)          # satisfied at once
        _lib.check_status()
        x = bf(64, 128)
        check(ops.rms_norm(x, torch.ones(128, device=DEV, dtype=torch.bfloat16)), ref.rms_norm(x.float(), torch.ones(128, device=DEV)), 1e-2)
    finally:
        _lib.set_peer_wait_ms(10000)
