"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op (GPU only)."""
import math

import pytest
import torch

from dew_b200 import ops
from dew_b200.ops import library as L
from dew_b200.ops.selection import KernelRefused

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def bf16_floor(ref, other_rounding=None):
    """RMS error of rounding the fp32 reference to bf16: the error any bf16-output kernel must carry."""
    return rel_err(ref.to(torch.bfloat16), ref)


@pytest.fixture(autouse=True)
def _status():
    yield
    L.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (130, 264, 72), (1000, 520, 392),
                                   (4096, 4096, 4096), (64, 128, 4096), (8, 256, 128)])
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_gemm_layouts(M, N, K, layout):
    torch.manual_seed(M * 7 + N * 3 + K)
    a_mn = layout == "tn"
    b_mn = layout in ("nn", "tn")
    A = torch.randn((K, M) if a_mn else (M, K), device=DEV).to(torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device=DEV).to(torch.bfloat16)
    if (a_mn and M % 8) or (b_mn and N % 8) or K % 8:
        with pytest.raises(KernelRefused):      # a row stride that breaks the 16-byte TMA rule is refused, not run
            ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, kernel="sm100_tcgen05")
        return
    out = ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, kernel="sm100_tcgen05")
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    assert out.shape == (M, N)
    err, floor = rel_err(out, ref), bf16_floor(ref)
    assert err <= 1.5 * floor + 1e-6, (err, floor)


@pytest.mark.parametrize("out_dtype,accumulate", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, True)])
def test_gemm_epilogues(out_dtype, accumulate):
    torch.manual_seed(3)
    M, N, K = 300, 520, 200
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    B = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    base = torch.randn(M, N, device=DEV).to(out_dtype)
    out = base.clone()
    ops.gemm(A, B, out=out, accumulate=accumulate, alpha=0.5, kernel="sm100_tcgen05")
    ref = 0.5 * (A.float() @ B.float().t()) + (base.float() if accumulate else 0)
    tol = 1e-5 if out_dtype == torch.float32 else 1.5 * bf16_floor(ref) + 1e-6
    assert rel_err(out, ref) <= tol


def test_gemm_canary_bounds():
    """Output rows / columns beyond (M, N) must not be touched: the output is a window inside a larger buffer."""
    torch.manual_seed(5)
    M, N, K = 200, 264, 136
    A = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    B = torch.randn(N, K, device=DEV).to(torch.bfloat16)
    big = torch.full((M + 64, N + 24), 7.0, device=DEV, dtype=torch.bfloat16)
    window = big[:M, :N]
    ops.gemm(A, B, out=window, kernel="sm100_tcgen05")
    assert torch.all(big[M:] == 7.0) and torch.all(big[:, N:] == 7.0)
    ref = A.float() @ B.float().t()
    assert rel_err(window, ref) <= 1.5 * bf16_floor(ref) + 1e-6


def test_gemm_deterministic():
    A = torch.randn(512, 1024, device=DEV).to(torch.bfloat16)
    B = torch.randn(768, 1024, device=DEV).to(torch.bfloat16)
    a = ops.gemm(A, B, kernel="sm100_tcgen05")
    b = ops.gemm(A, B, kernel="sm100_tcgen05")
    assert torch.equal(a, b)


def test_linear_autograd_matches_reference():
    torch.manual_seed(0)
    x = torch.randn(4, 96, 256, device=DEV).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(384, 256, device=DEV) / 16).to(torch.bfloat16).requires_grad_()
    y = ops.linear(x, w)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf @ wf.t()
    yf.backward(dy.float())
    assert rel_err(y, yf) <= 1.5 * bf16_floor(yf) + 1e-6
    assert rel_err(x.grad, xf.grad) <= 1.5 * bf16_floor(xf.grad) + 1e-6
    assert rel_err(w.grad, wf.grad) <= 1.5 * bf16_floor(wf.grad) + 1e-6


@pytest.mark.parametrize("rows,d", [(64, 128), (37, 1000), (512, 4096), (9, 8192)])
def test_rmsnorm_family(rows, d):
    torch.manual_seed(rows + d)
    x = torch.randn(rows, d, device=DEV).to(torch.bfloat16).requires_grad_()
    b = torch.randn(rows, d, device=DEV).to(torch.bfloat16).requires_grad_()
    w = (1 + 0.1 * torch.randn(d, device=DEV)).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, d, device=DEV).to(torch.bfloat16)
    # plain
    y = ops.rms_norm(x, w, 1e-6)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    yf.backward(dy.float())
    assert rel_err(y, yf) <= 2 * bf16_floor(yf)
    assert rel_err(x.grad, xf.grad) <= 2 * bf16_floor(xf.grad) + 1e-3
    assert rel_err(w.grad, wf.grad) <= 2e-2
    # stream: h = x + b, y = norm(h)
    x.grad = None; w.grad = None
    y2, h2 = ops.stream_rms_norm(x, b, w, 1e-6)
    (y2.float() * dy.float()).sum().backward()
    hf = (x.detach().float() + b.detach().float()).to(torch.bfloat16).float()
    assert torch.equal(h2.float(), hf)
    yf2 = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.detach().float()
    assert rel_err(y2, yf2) <= 2 * bf16_floor(yf2)
    assert torch.equal(x.grad, b.grad)
    # gated
    z = torch.randn(rows, d, device=DEV).to(torch.bfloat16).requires_grad_()
    x.grad = None; w.grad = None
    y3 = ops.gated_rms_norm(x, z, w, 1e-6)
    y3.backward(dy)
    xf, zf, wf = (t.detach().float().requires_grad_() for t in (x, z, w))
    yf3 = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf * torch.nn.functional.silu(zf)
    yf3.backward(dy.float())
    assert rel_err(y3, yf3) <= 2 * bf16_floor(yf3)
    assert rel_err(x.grad, xf.grad) <= 2 * bf16_floor(xf.grad) + 1e-3
    assert rel_err(z.grad, zf.grad) <= 2 * bf16_floor(zf.grad) + 1e-3


@pytest.mark.parametrize("rows,F", [(33, 64), (256, 14336), (1000, 1408)])
def test_packed_swiglu(rows, F):
    torch.manual_seed(F)
    gu = torch.randn(rows, 2 * F, device=DEV).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, F, device=DEV).to(torch.bfloat16)
    y = ops.packed_swiglu(gu)
    y.backward(dy)
    gf = gu.detach().float().requires_grad_()
    yf = torch.nn.functional.silu(gf[:, :F]) * gf[:, F:]
    yf.backward(dy.float())
    assert rel_err(y, yf) <= 2 * bf16_floor(yf)
    assert rel_err(gu.grad, gf.grad) <= 2 * bf16_floor(gf.grad) + 1e-3


def test_rope_roundtrip_and_reference():
    torch.manual_seed(1)
    B, S, H, D = 2, 48, 6, 128
    x = torch.randn(B, S, H, D, device=DEV).to(torch.bfloat16).requires_grad_()
    cos, sin = ops.rope_tables(64, D, 10000.0, DEV)
    y = ops.rope(x, cos, sin, rot_heads=4)
    ref = ops.rope_reference(x.detach().float(), cos, sin, None, 4)
    assert rel_err(y, ref) <= 2 * bf16_floor(ref)
    assert torch.equal(y[:, :, 4:], x.detach()[:, :, 4:])
    dy = torch.randn_like(y)
    y.backward(dy)
    xf = x.detach().float().requires_grad_()
    ops.rope_reference(xf, cos, sin, None, 4).backward(dy.float())
    assert rel_err(x.grad, xf.grad) <= 2 * bf16_floor(xf.grad) + 1e-3


@pytest.mark.parametrize("T,d,V,chunk", [(96, 64, 1000, 40), (300, 128, 5008, 128)])
def test_linear_cross_entropy(T, d, V, chunk):
    torch.manual_seed(T)
    h = torch.randn(T, d, device=DEV).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(V, d, device=DEV) / math.sqrt(d)).to(torch.bfloat16).requires_grad_()
    tg = torch.randint(0, V, (T,), device=DEV)
    tg[::7] = -100
    total, mass = ops.linear_cross_entropy(h, w, tg, z_loss=1e-4, chunk=chunk)
    (total / mass).backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rt, rm = ops.linear_cross_entropy_reference(hf, wf, tg, z_loss=1e-4)
    (rt / rm).backward()
    assert int(mass) == int(rm)
    assert abs(float(total) - float(rt)) / float(rt) < 5e-3
    assert rel_err(h.grad, hf.grad) < 3e-2
    assert rel_err(w.grad, wf.grad) < 3e-2


def test_adamw_and_grad_norm_match_torch():
    torch.manual_seed(2)
    n = 100_003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV).to(torch.bfloat16)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    pb = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    clip = torch.zeros(3, device=DEV)
    scratch = torch.empty(1024, device=DEV)
    for step in range(1, 4):
        ops.grad_norm_(g, clip, scratch, max_norm=1.0)
        ops.adamw_(p, m, v, g, step=step, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, p_bf16=pb, clip=clip)
        ref.grad = g.float().clone()
        torch.nn.utils.clip_grad_norm_([ref], 1.0)
        opt.step()
    assert abs(float(clip[1]) - float(g.float().norm())) / float(g.float().norm()) < 1e-4
    assert rel_err(p, ref.detach()) < 1e-5
    assert torch.equal(pb, p.to(torch.bfloat16))


def test_attention_matches_reference():
    torch.manual_seed(4)
    B, S, Hq, Hkv, D = 2, 256, 8, 2, 128
    q = torch.randn(B, S, Hq, D, device=DEV).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device=DEV).to(torch.bfloat16)
    out = ops.attention(q, k, v, causal=True)
    ref = ops.attention_reference(q.float(), k.float(), v.float(), causal=True)
    assert rel_err(out, ref) <= 3 * bf16_floor(ref) + 1e-3


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 128, 1, 1, 128, True), (2, 256, 8, 2, 128, True), (1, 512, 4, 4, 128, False),
                                                 (2, 384, 4, 2, 64, True), (1, 1024, 2, 1, 128, True)])
@pytest.mark.parametrize("variant", [1, 0])
def test_flash_forward_sm100(B, S, Hq, Hkv, D, causal, variant, flash_variant):
    """variant 1 keeps P in tensor memory (the default), 0 passes it through shared memory."""
    from dew_b200.ops.flash import flash_fwd
    flash_variant(variant)
    torch.manual_seed(S + D)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV).to(torch.bfloat16)      # packed projection layout
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    out, lse = flash_fwd(q, k, v, causal, 1.0 / math.sqrt(D))
    ref = ops.attention_reference(q.float(), k.float(), v.float(), causal=causal)
    assert rel_err(out, ref) <= 3 * bf16_floor(ref) + 2e-3, rel_err(out, ref)
    rep = Hq // Hkv
    s = torch.einsum("bshd,bthd->bhst", q.float(), k.float().repeat_interleave(rep, 2)) / math.sqrt(D)
    if causal:
        s = s.masked_fill(~torch.tril(torch.ones(S, S, dtype=torch.bool, device=DEV)), float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=2e-2, rtol=1e-3)


@pytest.fixture
def flash_variant():
    """Selects the forward variant for one test and restores the previous one afterwards."""
    lib = L.load()
    previous = []

    def select(v):
        previous.append(lib.dewb_flash_set_variant(int(v)))
    yield select
    if previous:
        lib.dewb_flash_set_variant(previous[0])


@pytest.mark.parametrize("variant", [1, 0])
def test_flash_forward_large_values_rescale(variant, flash_variant):
    """Rows whose maximum grows tile after tile exercise the lazy rescale of the TMEM accumulator."""
    from dew_b200.ops.flash import flash_fwd
    flash_variant(variant)
    torch.manual_seed(9)
    B, S, H, D = 1, 512, 2, 128
    q = torch.randn(B, S, H, D, device=DEV).to(torch.bfloat16)
    k = (torch.randn(B, S, H, D, device=DEV) * torch.linspace(0.5, 6.0, S, device=DEV)[None, :, None, None]).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, device=DEV).to(torch.bfloat16)
    out, _ = flash_fwd(q, k, v, True, 1.0 / math.sqrt(D))
    ref = ops.attention_reference(q.float(), k.float(), v.float(), causal=True)
    assert rel_err(out, ref) <= 3 * bf16_floor(ref) + 2e-3, rel_err(out, ref)


@pytest.mark.parametrize("B,S,Hq,Hkv,D,causal", [(1, 128, 1, 1, 128, True), (2, 256, 4, 2, 128, True), (1, 384, 2, 2, 128, False),
                                                 (1, 256, 4, 1, 64, True), (1, 1024, 4, 2, 128, True)])
def test_flash_backward_sm100(B, S, Hq, Hkv, D, causal):
    torch.manual_seed(S * 3 + D)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV).to(torch.bfloat16).requires_grad_()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    out = ops.attention(q, k, v, causal=causal, kernel="sm100_flash")
    do = torch.randn_like(out)
    out.backward(do)
    got = qkv.grad.clone()
    ref_in = qkv.detach().float().requires_grad_()
    rq, rk, rv = ref_in[:, :, :Hq], ref_in[:, :, Hq:Hq + Hkv], ref_in[:, :, Hq + Hkv:]
    ref = ops.attention_reference(rq, rk, rv, causal=causal)
    ref.backward(do.float())
    for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
        g, r = got[:, :, sl], ref_in.grad[:, :, sl]
        assert rel_err(g, r) <= 3 * bf16_floor(r) + 1.5e-2, (name, rel_err(g, r))


@pytest.mark.parametrize("M,N,K,a_mn,b_mn,dtype,acc", [
    (512, 512, 256, False, False, torch.bfloat16, False), (384, 768, 192, False, True, torch.bfloat16, False),
    (304, 520, 136, True, True, torch.float32, True), (1024, 256, 64, True, False, torch.float32, False),
    (2048, 4096, 1024, False, False, torch.bfloat16, True)])
def test_gemm_pair_kernel_matches_reference(M, N, K, a_mn, b_mn, dtype, acc):
    """The CTA-pair (cta_group::2) kernel: every operand layout, epilogue, odd sizes with row / column / reduction tails."""
    torch.manual_seed(M + N + K)
    A = torch.randn((K, M) if a_mn else (M, K), device=DEV).to(torch.bfloat16)
    B = torch.randn((K, N) if b_mn else (N, K), device=DEV).to(torch.bfloat16)
    pad = torch.full((M + 2, N), 7.0, device=DEV, dtype=dtype)          # canary rows after the output
    out = pad[:M]
    if acc:
        out.normal_()
    before = out.float().clone()
    ops.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=acc, kernel="sm100_pair")
    L.check_status()
    ref = (A.float().t() if a_mn else A.float()) @ (B.float() if b_mn else B.float().t())
    if acc:
        ref = ref + before
    assert rel_err(out, ref) <= 2 * bf16_floor(ref) + 1e-5, rel_err(out, ref)
    assert bool((pad[M:] == 7.0).all())


@pytest.mark.parametrize("B,S,Hq,Hkv,D", [(2, 256, 4, 2, 128), (1, 512, 8, 2, 64)])
def test_packed_rope_flash_matches_unfused_reference(B, S, Hq, Hkv, D):
    """One autograd node for RoPE + attention over the packed projection (in-place rotation, packed gradient buffer)
    against fp32 rope + attention through plain autograd."""
    from dew_b200.ops.attn import packed_attention
    torch.manual_seed(B * S + D)
    cos, sin = ops.rope_tables(S, D, 10000.0, device=DEV)
    base = torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV).to(torch.bfloat16)
    x = base.clone().requires_grad_()
    out = packed_attention(x * 1.0, cos, sin, None, Hq, Hkv, True)          # `* 1.0`: a fresh tensor the op may rotate in place
    assert out is not None
    do = torch.randn_like(out)
    out.backward(do)
    ref_in = base.float().requires_grad_()
    r = ops.rope_reference(ref_in, cos, sin, None, Hq + Hkv)
    ref = ops.attention_reference(r[:, :, :Hq], r[:, :, Hq:Hq + Hkv], r[:, :, Hq + Hkv:], causal=True)
    ref.backward(do.float())
    assert rel_err(out, ref) <= 3 * bf16_floor(ref) + 3e-3, rel_err(out, ref)
    for name, sl in (("dq", slice(0, Hq)), ("dk", slice(Hq, Hq + Hkv)), ("dv", slice(Hq + Hkv, None))):
        g, rr = x.grad[:, :, sl], ref_in.grad[:, :, sl]
        assert rel_err(g, rr) <= 3 * bf16_floor(rr) + 1.5e-2, (name, rel_err(g, rr))


@pytest.mark.parametrize("T,k,E,d,F", [(300, 2, 4, 128, 192), (1000, 6, 16, 256, 128), (64, 2, 8, 64, 64)])
def test_grouped_gemm_forward_backward(T, k, E, d, F):
    """tcgen05 grouped GEMMs (expert-sorted, 128-aligned groups) against the per-expert fp32 loop."""
    from dew_b200.ops import grouped as G
    torch.manual_seed(T + E)
    ids = torch.randint(0, E, (T, k), device=DEV)
    if E > 4:
        ids[ids == 3] = 2                                     # leave one expert empty
    layout = G.group_layout(ids, E)
    x = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    xs = G.permute(x, layout, k).requires_grad_()
    w = (torch.randn(E, F, d, device=DEV) / math.sqrt(d)).to(torch.bfloat16).requires_grad_()
    y = G.grouped_linear(xs, w, layout)
    dy = torch.randn_like(y)
    # padding rows carry no gradient in a real layer (combine never reads them)
    used = torch.zeros(layout.rows, dtype=torch.bool, device=DEV)
    used[layout.positions] = True
    dy = dy * used[:, None]
    y.backward(dy)
    ref_y = G._gmm_reference(xs.detach(), w.detach(), layout, False)
    assert rel_err(y[used], ref_y[used].float()) <= 1e-2
    ref_dx = G._gmm_reference(dy, w.detach(), layout, True)
    assert rel_err(xs.grad[used], ref_dx[used].float()) <= 1e-2
    ref_dw = G._tgmm_reference(dy, xs.detach(), layout, E)
    assert rel_err(w.grad, ref_dw) <= 1e-2
    assert torch.all(y[~used] == 0)                           # zero rows in, zero rows out


@pytest.mark.parametrize("quantized,page_size,D,Hq,Hkv", [(None, 16, 128, 8, 2), (None, 64, 128, 4, 1), ("int8", 16, 128, 8, 2),
                                                          ("float8_e4m3fn", 32, 64, 4, 4), (None, None, 128, 32, 8),
                                                          (None, 64, 128, 32, 8), (None, 128, 128, 8, 1), (None, 64, 128, 6, 2)])
def test_paged_decode_attention(quantized, page_size, D, Hq, Hkv):
    from dew_b200.nn.kv_cache import KVCache, KVStore, paged_attention_reference
    torch.manual_seed(11)
    rows, max_len = 6, 700
    store = KVStore(KVCache(quantized=quantized, page_size=page_size), 1, rows, max_len, Hkv, D, torch.bfloat16, DEV)
    if page_size:                                   # scatter the pages so the table matters
        perm = torch.randperm(store.pages, device=DEV).to(torch.int32)
        store.page_table.copy_(perm.reshape(rows, store.max_pages))
    lengths = torch.tensor([1, 17, 256, 511, 640, 699], device=DEV, dtype=torch.int32)
    S = int(lengths.max())
    k = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
    pos = torch.arange(S, device=DEV)[None].expand(rows, S).clone()
    pos[pos >= lengths[:, None]] = -1
    store.write(0, k, v, pos)
    # one more token through the append kernel
    k1 = torch.randn(rows, Hkv, D, device=DEV).to(torch.bfloat16)
    v1 = torch.randn(rows, Hkv, D, device=DEV).to(torch.bfloat16)
    store.append(0, k1, v1, lengths)
    lengths = lengths + 1
    q = torch.randn(rows, Hq, D, device=DEV).to(torch.bfloat16)
    out = store.decode_attention(0, q, lengths)
    ref = paged_attention_reference(store, 0, q.float(), lengths, 1.0 / math.sqrt(D))
    assert rel_err(out, ref) <= 2e-2, rel_err(out, ref)


def test_paged_decode_streamed_kernel_window_sinks_and_long_rows():
    """The TMA-streamed decode kernel (64-key pages, bf16) with a sliding window, attention sinks and rows long enough for
    several key splits, against the reference; and against the first-generation kernel on the same store."""
    import os
    from dew_b200.nn.kv_cache import KVCache, KVStore, paged_attention_reference
    torch.manual_seed(5)
    rows, max_len, Hq, Hkv, D = 9, 2304, 32, 8, 128
    store = KVStore(KVCache(page_size=64), 1, rows, max_len, Hkv, D, torch.bfloat16, DEV)
    perm = torch.randperm(store.pages, device=DEV).to(torch.int32)
    store.page_table.copy_(perm.reshape(rows, store.max_pages))
    lengths = torch.tensor([1, 63, 64, 65, 500, 1024, 1500, 2303, 2304], device=DEV, dtype=torch.int32)
    S = int(lengths.max())
    k = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
    v = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
    pos = torch.arange(S, device=DEV)[None].expand(rows, S).clone()
    pos[pos >= lengths[:, None]] = -1
    store.write(0, k, v, pos)
    q = torch.randn(rows, Hq, D, device=DEV).to(torch.bfloat16)
    sinks = torch.randn(Hq, device=DEV)
    for window, sk in ((None, None), (300, None), (None, sinks), (1000, sinks)):
        out = store.decode_attention(0, q, lengths, window=window, sinks=sk)
        ref = paged_attention_reference(store, 0, q.float(), lengths, 1.0 / math.sqrt(D), window, sk, 0.0)
        assert rel_err(out, ref) <= 2e-2, (window, sk is not None, rel_err(out, ref))
        os.environ["DEWB_DECODE"] = "lanes"
        try:
            old = store.decode_attention(0, q, lengths, window=window, sinks=sk)
        finally:
            os.environ.pop("DEWB_DECODE")
        assert rel_err(out, old) <= 2e-2


@pytest.mark.parametrize("Hq,Hkv", [(4, 1), (32, 8)])
def test_paged_decode_balanced_persistent_kernel(Hq, Hkv):
    """The balanced persistent form of the streamed decode kernel (every CTA takes the same number of tiles; rows cut across
    CTAs are merged by the last one to arrive) on a serving-sized batch: 128 rows of very different lengths, some empty, against
    the reference and against the one-CTA-per-chunk form; twice, so that the self-resetting tickets are seen to reset."""
    import os
    from dew_b200.nn.kv_cache import KVCache, KVStore, paged_attention_reference
    torch.manual_seed(17)
    rows, max_len, D = 128, 2304, 128
    store = KVStore(KVCache(page_size=64), 1, rows, max_len, Hkv, D, torch.bfloat16, DEV)
    perm = torch.randperm(store.pages, device=DEV).to(torch.int32)
    store.page_table.copy_(perm.reshape(rows, store.max_pages))
    store.k.normal_()
    store.v.normal_()
    lengths = torch.randint(1, max_len + 1, (rows,), device=DEV, dtype=torch.int32)
    lengths[::17] = 0                                    # rows that hold nothing yet
    lengths[5], lengths[6] = 1, 2304
    q = torch.randn(rows, Hq, D, device=DEV).to(torch.bfloat16)
    sinks = torch.randn(Hq, device=DEV)
    for window, sk in ((None, None), (700, sinks)):
        ref = paged_attention_reference(store, 0, q.float(), lengths, 1.0 / math.sqrt(D), window, sk, 0.0)
        live = lengths > 0
        for _ in range(2):
            out = store.decode_attention(0, q, lengths, window=window, sinks=sk)
            assert rel_err(out[live], ref[live]) <= 2e-2, (window, rel_err(out[live], ref[live]))
            assert torch.all(out[~live] == 0)
        os.environ["DEWB_DECODE_PERSIST"] = "0"
        try:
            chunked = store.decode_attention(0, q, lengths, window=window, sinks=sk)
        finally:
            os.environ.pop("DEWB_DECODE_PERSIST")
        assert rel_err(chunked[live], ref[live]) <= 2e-2
    assert int(store._arrivals.abs().sum()) == 0
    L.check_status()


@pytest.mark.parametrize("B,T,C,K,act,bias", [(2, 200, 64, 4, True, False), (1, 1000, 4096 + 8, 4, True, True), (3, 65, 128, 3, False, True)])
def test_short_conv_forward_backward(B, T, C, K, act, bias):
    from dew_b200.ops import scan
    torch.manual_seed(T)
    x = torch.randn(B, T, C, device=DEV).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(C, K, device=DEV) * 0.5).requires_grad_()
    b = torch.randn(C, device=DEV).requires_grad_() if bias else None
    y = scan.short_conv(x, w, b, act)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    bf = b.detach().clone().requires_grad_() if bias else None
    ref = scan.short_conv_reference(xf, wf, bf, act)
    ref.backward(dy.float())
    assert rel_err(y, ref) <= 2 * bf16_floor(ref) + 1e-3
    assert rel_err(x.grad, xf.grad) <= 2 * bf16_floor(xf.grad) + 2e-3
    assert rel_err(w.grad, wf.grad) <= 1e-2
    if bias:
        assert rel_err(b.grad, bf.grad) <= 1e-2


@pytest.mark.parametrize("T,E,k,fn,norm,with_bias", [(1000, 64, 6, "softmax", True, False), (333, 8, 2, "softmax", False, True),
                                                      (512, 160, 8, "sigmoid", True, True), (64, 256, 1, "softmax", False, False)])
def test_moe_route_kernel(T, E, k, fn, norm, with_bias):
    from dew_b200.ops.routing import route, _formula
    torch.manual_seed(T + E)
    logits = (torch.randn(T, E, device=DEV) * 2).requires_grad_()
    bias = torch.randn(E, device=DEV) * 0.01 if with_bias else None
    w, ids, scores = route(logits, bias, k, fn, norm, 1.5)
    ref_scores = torch.softmax(logits, -1) if fn == "softmax" else torch.sigmoid(logits)
    sel = ref_scores + bias if with_bias else ref_scores
    ref_ids = torch.topk(sel, k, dim=-1).indices
    assert torch.equal(ids.sort(-1).values, ref_ids.sort(-1).values)
    assert torch.allclose(scores, ref_scores, atol=1e-6, rtol=1e-4)
    ref_w, _ = _formula(logits, ids, fn, norm, 1.5)
    assert torch.allclose(w, ref_w, atol=1e-6, rtol=1e-4)
    dw, dsc = torch.randn_like(w), torch.randn_like(scores)
    (g,) = torch.autograd.grad((w, scores), logits, (dw, dsc))
    lg = logits.detach().clone().requires_grad_()
    rw, rs = _formula(lg, ids, fn, norm, 1.5)
    (rg,) = torch.autograd.grad((rw, rs), lg, (dw, dsc))
    assert torch.allclose(g, rg, atol=1e-6, rtol=1e-4)


@pytest.mark.parametrize("T,d,E,k", [(300, 256, 8, 2), (1024, 512, 64, 6), (77, 128, 16, 4)])
def test_moe_token_exchange_single_rank(T, d, E, k):
    """plan / push / pull kernels with this rank as its own peer against the index arithmetic in PyTorch."""
    from dew_b200.ops import grouped as G
    from dew_b200.parallel.ep import TokenExchange
    torch.manual_seed(T)
    x = torch.randn(T, d, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)])
    w = torch.rand(T, k, device=DEV)
    ex = TokenExchange(E, "self")
    plan = ex.plan(ids, d)
    ref = G.group_layout(ids.reshape(-1), E)
    assert int(plan.info[1]) == 0 and int(plan.info[0]) == int(ref.offsets[-1])
    assert torch.equal(plan.layout.offsets, ref.offsets) and torch.equal(plan.layout.counts, ref.counts)
    assert torch.equal(plan.layout.tile_group, ref.tile_group)
    assert torch.equal(plan.dest_pos.long(), ref.positions) and int(plan.dest_rank.abs().max()) == 0
    rows = ex.push(x, plan)
    assert torch.equal(rows, G.permute(x, ref, k))
    y = torch.randn_like(rows)
    out, kept = ex.pull(y, plan, w, keep_rows=True)
    assert rel_err(out, G.combine(y, ref, w, T)) <= 1e-2
    assert torch.equal(kept, y.index_select(0, ref.positions))
    scaled = ex.push(x, plan, pair_scale=w.reshape(-1))
    want = torch.zeros_like(rows).index_copy(0, ref.positions, (x.float().repeat_interleave(k, 0) * w.reshape(-1, 1)).to(torch.bfloat16))
    assert rel_err(scaled, want) <= 1e-2


def test_sparse_mlp_exchange_path_matches_index_path():
    """The mixture layer on the routing / exchange kernels against the same layer on PyTorch index ops (outputs, gradients)."""
    from dew_b200.models.causal_transformer import Mixture
    from dew_b200.nn import moe as M
    mix = Mixture(experts=16, top_k=4, expert_features=128, shared_features=128)
    torch.manual_seed(0)
    a = M.SparseMLP(256, mix, 512).to(DEV, torch.bfloat16)
    torch.manual_seed(0)
    b = M.SparseMLP(256, mix, 512).to(DEV, torch.bfloat16)
    b.use_kernels = False
    x = torch.randn(2, 300, 256, device=DEV).to(torch.bfloat16)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, yb = a(xa), b(xb)
    assert rel_err(ya, yb) <= 2e-2
    dy = torch.randn_like(ya)
    ya.backward(dy)
    yb.backward(dy)
    assert rel_err(xa.grad, xb.grad) <= 3e-2
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert rel_err(pa.grad, pb.grad) <= 5e-2, n


@pytest.mark.parametrize("B,T,H,D,strided", [(2, 100, 4, 128, True), (1, 333, 3, 64, False), (2, 50, 2, 256, True)])
def test_l2_normalize_kernel(B, T, H, D, strided):
    torch.manual_seed(T)
    wide = torch.randn(B, T, 3 * H * D + 8, device=DEV).to(torch.bfloat16)
    src = wide[..., 8:8 + H * D] if strided else wide[..., :H * D].contiguous()
    x = src.reshape(B, T, H, D).detach().requires_grad_()
    y = ops.l2_normalize(x)
    assert y.dtype == torch.bfloat16 and y.is_contiguous()
    dy = torch.randn_like(y)
    y.backward(dy)
    xf = x.detach().float().requires_grad_()
    ref = torch.nn.functional.normalize(xf, dim=-1)
    ref.backward(dy.float())
    assert rel_err(y, ref) <= 2 * bf16_floor(ref)
    assert rel_err(x.grad, xf.grad) <= 2e-2


def test_gated_delta_net_layer_gpu_matches_cpu_reference():
    """The whole mixer (projections, short conv, l2-norm, gated delta rule kernels, gated norm) on the GPU in bf16 against the
    same module in fp32 on the CPU."""
    from dew_b200.nn.linear_attention import GatedDeltaNet
    torch.manual_seed(0)
    ref = GatedDeltaNet(256, num_k_heads=2, num_v_heads=2, head_k_dim=128, head_v_dim=128)
    gpu = GatedDeltaNet(256, num_k_heads=2, num_v_heads=2, head_k_dim=128, head_v_dim=128)
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.to(DEV)
    for n, p in gpu.named_parameters():
        if n not in ("A_log", "dt_bias"):
            p.data = p.data.to(torch.bfloat16)
    x = torch.randn(2, 200, 256) * 0.5
    xr = x.clone().requires_grad_()
    xg = x.to(DEV, torch.bfloat16).requires_grad_()
    yr, yg = ref(xr), gpu(xg)
    assert rel_err(yg.cpu(), yr) <= 5e-2
    dy = torch.randn_like(yr)
    yr.backward(dy)
    yg.backward(dy.to(DEV, torch.bfloat16))
    assert rel_err(xg.grad.cpu(), xr.grad) <= 8e-2
    assert rel_err(gpu.A_log.grad.cpu(), ref.A_log.grad) <= 8e-2
    assert rel_err(gpu.in_proj_qkvz.weight.grad.cpu(), ref.in_proj_qkvz.weight.grad) <= 8e-2


@pytest.mark.parametrize("V,dtype", [(1000, torch.float32), (128256, torch.bfloat16), (32768, torch.float32)])
def test_argmax_rows_kernel(V, dtype):
    from dew_b200.ops import sample as S
    torch.manual_seed(V)
    x = torch.randn(7, V, device=DEV).to(dtype)
    x[3, 5] = x[3, 900] = 50.0                                   # a tie: the lower index wins
    got = S.argmax_rows(x)
    want = torch.stack([torch.nonzero(r == r.max())[0, 0] for r in x.float()])
    assert torch.equal(got, want)


@pytest.mark.parametrize("V,temperature,top_k,top_p,min_p", [(1000, 1.0, None, 1.0, 0.0), (5000, 0.7, 50, 1.0, 0.0),
                                                            (128256, 1.3, None, 0.9, 0.0), (32768, 0.8, 200, 0.95, 0.02),
                                                            (777, 1.0, 5, 0.5, 0.0)])
def test_sample_rows_kernel_filters_and_inverse_cdf(V, temperature, top_k, top_p, min_p):
    """The kept set equals the thresholds' set, and the drawn token is the inverse CDF of the filtered distribution at u."""
    from dew_b200.ops import sample as S
    torch.manual_seed(V)
    R = 16
    logits = torch.randn(R, V, device=DEV) * 3
    u = torch.rand(R, device=DEV)
    tok, kept = S.sample_rows(logits, u, temperature, top_k, top_p, min_p, return_kept=True)
    ref = S.filtered_reference(logits, temperature, top_k, top_p, min_p)
    ref_kept = torch.isfinite(ref).sum(-1)
    assert (kept.long() - ref_kept).abs().max() <= 1             # a threshold may fall between two nearly equal masses
    assert torch.isfinite(ref.gather(-1, tok[:, None])).all()    # every draw is a kept token
    e = torch.exp(ref.double() - ref.double().max(-1, keepdim=True).values)
    cdf = e.cumsum(-1) / e.sum(-1, keepdim=True)
    hi = cdf.gather(-1, tok[:, None])[:, 0]
    lo = hi - (e / e.sum(-1, keepdim=True)).gather(-1, tok[:, None])[:, 0]
    same_set = kept.long() == ref_kept
    assert ((u.double() >= lo - 1e-4) & (u.double() <= hi + 1e-4))[same_set].all()


def test_sample_rows_kernel_distribution():
    from dew_b200.ops import sample as S
    torch.manual_seed(0)
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 3.0, -30.0]], device=DEV).repeat(20000, 1)
    tok = S.sample_rows(logits, torch.rand(20000, device=DEV), 1.0, 4, 1.0, 0.0)
    freq = torch.bincount(tok, minlength=6).float() / 20000
    want = torch.softmax(torch.tensor([2.0, 1.0, 0.0, float("-inf"), 3.0, float("-inf")]), -1).to(DEV)
    assert (freq - want).abs().max() < 0.015


@pytest.mark.parametrize("B,T,H,G,with_state", [(1, 64, 2, 1, False), (2, 300, 4, 2, True), (1, 1024, 8, 1, False)])
def test_ssd_scan_kernel_against_recurrent_oracle(B, T, H, G, with_state):
    from dew_b200.ops import scan
    torch.manual_seed(T + H)
    x = torch.randn(B, T, H, 64, device=DEV).to(torch.bfloat16)
    dt = torch.nn.functional.softplus(torch.randn(B, T, H, device=DEV) - 2)
    A = -torch.rand(H, device=DEV) * 4 - 0.5
    Bm = (torch.randn(B, T, G, 128, device=DEV) / 8).to(torch.bfloat16)
    Cm = (torch.randn(B, T, G, 128, device=DEV) / 8).to(torch.bfloat16)
    D = torch.randn(H, device=DEV)
    s0 = torch.randn(B, H, 64, 128, device=DEV) * 0.2 if with_state else None
    leaves = [t.clone().requires_grad_() for t in (x, dt, Bm, Cm)]
    y, S = scan.ssd(leaves[0], leaves[1], A, leaves[2], leaves[3], D, s0)
    ref_leaves = [t.detach().float().requires_grad_() for t in leaves]
    ry, rS = scan.ssd_recurrent(ref_leaves[0], ref_leaves[1], A, ref_leaves[2], ref_leaves[3], D, s0)
    assert rel_err(y, ry) <= 2e-2 and rel_err(S, rS) <= 2e-2
    dy = torch.randn_like(y)
    y.backward(dy)
    ry.backward(dy.float())
    for name, a, b in zip(("dx", "ddt", "dB", "dC"), leaves, ref_leaves):
        assert rel_err(a.grad, b.grad) <= 4e-2, (name, rel_err(a.grad, b.grad))


def _gdn_inputs(B, T, H, seed, with_state):
    torch.manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, 128, device=DEV), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, 128, device=DEV), dim=-1).to(torch.bfloat16)
    v = torch.randn(B, T, H, 128, device=DEV).to(torch.bfloat16)
    g = -torch.rand(B, T, H, device=DEV) * 0.3
    beta = torch.rand(B, T, H, device=DEV)
    s0 = torch.randn(B, H, 128, 128, device=DEV) * 0.1 if with_state else None
    return q, k, v, g, beta, s0


@pytest.mark.parametrize("B,T,H,with_state", [(1, 64, 1, False), (2, 300, 3, True), (1, 1024, 2, False)])
def test_gdn_kernel_stages_match_their_restatements(B, T, H, with_state):
    """Each of the three gated-delta-rule kernels against the PyTorch restatement of the same stage (fp32)."""
    from dew_b200.ops import gdn
    q, k, v, g, beta, s0 = _gdn_inputs(B, T, H, T, with_state)
    scale = 128 ** -0.5
    gc, W, U, P, Qg = gdn.prepare_cuda(q, k, v, g, beta, scale, True)
    rgc, rW, rU, rP, rQg = gdn.prepare_reference(q.float(), k.float(), v.float(), g, beta, scale)
    assert torch.allclose(gc, rgc, atol=1e-4)
    for got, ref in ((W, rW), (U, rU), (P, rP), (Qg, rQg)):
        assert rel_err(got, ref) <= 2 * bf16_floor(ref) + 1e-3
    # the scans, fed the kernel's own (bf16) intermediates so that only the scan is under test
    o, final, states = gdn.scan_fwd_cuda(q, k, gc, W, U, P, scale, s0, True)
    ro, rfinal, rstates = gdn.scan_fwd_reference(q.float(), k.float(), gc, W.float(), U.float(), P.float(), scale, s0, True)
    assert rel_err(o, ro) <= 2e-2
    assert rel_err(final, rfinal) <= 2e-2
    assert rel_err(states, rstates) <= 2e-2
    do = torch.randn(B, T, H, 128, device=DEV).to(torch.bfloat16)
    dfin = torch.randn(B * H, 128, 128, device=DEV) * 0.1 if with_state else None
    ds, dinit = gdn.scan_bwd_cuda(do, k, gc, W, P, Qg, dfin)
    rds, rdinit = gdn.scan_bwd_reference(do.float(), k.float(), gc, W.float(), P.float(), Qg.float(), dfin)
    assert rel_err(ds, rds) <= 2e-2
    assert rel_err(dinit, rdinit) <= 2e-2


def test_gdn_shared_key_heads_match_repeated_heads():
    """Two value heads per key head read the key head in place: same outputs and gradients as with q, k repeated."""
    from dew_b200.ops import scan
    B, T, Hk, rep = 2, 200, 2, 2
    q, k, v, g, beta, _ = _gdn_inputs(B, T, Hk * rep, 11, False)
    q, k = q[:, :, :Hk].contiguous(), k[:, :, :Hk].contiguous()
    a = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    b = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
    oa, Sa = scan.chunk_gated_delta_rule(*a)
    ob, Sb = scan.chunk_gated_delta_rule(b[0].repeat_interleave(rep, 2), b[1].repeat_interleave(rep, 2), *b[2:])
    assert torch.equal(oa, ob) and torch.equal(Sa, Sb)
    do = torch.randn_like(oa)
    oa.backward(do)
    ob.backward(do)
    for name, x, y in zip(("dq", "dk", "dv", "dg", "dbeta"), a, b):
        assert rel_err(x.grad, y.grad) <= 1e-2, (name, rel_err(x.grad, y.grad))


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 300, 2), (1, 1024, 3)])
def test_gdn_local_backward_kernels_match_closed_form(B, T, H):
    """The two chunk-local backward kernels against the closed-form gradients in PyTorch, both fed the same
    intermediates (entry states, exit-state gradients, Vn, dVn) from the scan kernels."""
    from dew_b200.ops import gdn
    q, k, v, g, beta, s0 = _gdn_inputs(B, T, H, 7 * T, True)
    scale = 128 ** -0.5
    do = torch.randn(B, T, H, 128, device=DEV).to(torch.bfloat16)
    gc, W, U, P, Qg = gdn.prepare_cuda(q, k, v, g, beta, scale, True)
    _, _, states_raw, vn = gdn.scan_fwd_cuda(q, k, gc, W, U, P, scale, s0, True, save_vn=True)
    dstates16, dvn, _ = gdn.scan_bwd_cuda(do, k, gc, W, P, Qg, None, for_kernels=True)
    got = gdn.local_bwd_cuda(q, k, v, do, gc, beta, W, U, P, vn, dvn, states_raw, dstates16, scale)
    L.check_status()
    ref = gdn.chunk_local_grads(q, k, v, g, beta, states_raw.transpose(-1, -2).float(), dstates16.float(), do, scale)
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta"), got, ref):
        assert torch.isfinite(a.float()).all(), name
        assert rel_err(a, b) <= 3e-2, (name, rel_err(a, b))


@pytest.mark.parametrize("B,T,H,with_state", [(2, 200, 2, True), (1, 512, 4, False)])
def test_gdn_forward_backward_against_recurrent_oracle(B, T, H, with_state):
    from dew_b200.ops import scan
    q, k, v, g, beta, s0 = _gdn_inputs(B, T, H, 100 + T, with_state)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)] + ([s0.clone().requires_grad_()] if with_state else [])
    o, S = scan.chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5] if with_state else None)
    do = torch.randn_like(o)
    dS = torch.randn_like(S) * 0.1
    torch.autograd.backward((o, S), (do, dS))
    ref_leaves = [t.detach().float().requires_grad_() for t in leaves]
    ro, rS = scan.gated_delta_rule_chunked(*ref_leaves[:5], initial_state=ref_leaves[5] if with_state else None)
    torch.autograd.backward((ro, rS), (do.float(), dS))
    assert rel_err(o, ro) <= 2e-2 and rel_err(S, rS) <= 2e-2
    for name, a, b in zip(("dq", "dk", "dv", "dg", "dbeta", "ds0"), leaves, ref_leaves):
        assert rel_err(a.grad, b.grad) <= 4e-2, (name, rel_err(a.grad, b.grad))


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 264, 1024), (4096, 4096, 4096)])
def test_fp8_rowwise_gemm(M, N, K):
    from dew_b200.ops import fp8
    torch.manual_seed(M)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    aq, asc = fp8.quantize_rows(a)
    bq, bsc = fp8.quantize_rows(b)
    # the quantiser itself: values round-trip within e4m3 precision, scales are absmax / 448
    assert torch.allclose(asc, a.float().abs().amax(-1) / 448.0, rtol=1e-3)
    out = fp8.gemm_fp8(aq, asc, bq, bsc)
    exact_q = (aq.float() * asc[:, None]) @ (bq.float() * bsc[:, None]).t()           # what the kernel must compute
    assert rel_err(out, exact_q) <= 1.5 * bf16_floor(exact_q) + 1e-4
    ref = a.float() @ b.float().t()
    assert rel_err(out, ref) < 0.06                                                   # fp8 quantisation error itself


def test_fp8_grouped_linear_matches_bf16_path():
    from dew_b200.ops import grouped as G
    from dew_b200.ops.fp8 import fp8_grouped_linear
    torch.manual_seed(5)
    T, k, E, d, F = 500, 2, 8, 256, 384
    ids = torch.randint(0, E, (T, k), device=DEV)
    layout = G.group_layout(ids, E)
    xs = G.permute(torch.randn(T, d, device=DEV).to(torch.bfloat16), layout, k).requires_grad_()
    w = (torch.randn(E, F, d, device=DEV) / math.sqrt(d)).to(torch.bfloat16).requires_grad_()
    y8 = fp8_grouped_linear(xs, w, layout)
    y16 = G.grouped_linear(xs.detach(), w.detach(), layout)
    used = torch.zeros(layout.rows, dtype=torch.bool, device=DEV)
    used[layout.positions] = True
    assert rel_err(y8[used], y16[used].float()) < 0.06
    (y8 * used[:, None]).sum().backward()
    assert xs.grad is not None and w.grad is not None and torch.isfinite(w.grad.float()).all()


@pytest.mark.parametrize("fisheye", [False, True])
def test_raycast_kernel_matches_cpu_restatement(fisheye):
    """The CUDA ray caster against the fp32 torch restatement of the same scene (gates, pillars, ground, sky, two shutter
    poses): pixels agree except where a ray grazes an edge and the nearest hit flips."""
    from dew_b200.rl import Camera, gate_boxes, look_at, render, render_reference
    torch.manual_seed(3)
    B = 3
    pos = torch.tensor([[0.0, 0.0, 1.4], [1.0, -2.0, 2.0], [-3.0, 0.5, 0.8]])
    tgt = torch.tensor([[5.0, 0.2, 1.5], [4.0, 1.0, 1.2], [2.0, 0.0, 1.6]])
    cams = torch.stack([look_at(pos, tgt), look_at(pos + 0.05, tgt)], 1)
    centers = torch.tensor([[[5.0, 0.0, 1.5], [8.0, 3.0, 1.8]]]).expand(B, 2, 3).contiguous()
    boxes = gate_boxes(centers, torch.tensor([[0.0, 0.7]]).expand(B, 2).contiguous()).reshape(B, 8, 10)
    cyl = torch.tensor([[[3.0, 2.0, 0.2, 3.0, 0.2, 0.3, 0.9], [6.0, -2.5, 0.4, 2.0, 0.9, 0.8, 0.1]]]).expand(B, 2, 7).contiguous()
    cam = Camera(size=(64, 80), fov=110.0, fisheye=fisheye, samples=2)
    ref = render_reference(cams, boxes, cyl, cam)
    got = render(cams.to(DEV), boxes.to(DEV), cyl.to(DEV), cam).cpu()
    close = (got - ref).abs().max(-1).values < 2e-3
    assert close.float().mean() > 0.995, float(close.float().mean())
    assert float((got - ref).abs().mean()) < 2e-3


def test_kernels_are_on_par_with_pytorch_bf16_against_float64():
    """The accuracy contract (``dew_b200.utils.parity``): over 8 seeds, each kernel's error from the float64 truth is within
    1.5x that of the same op computed by PyTorch in bf16, and its worst row within 4x, forward and backward."""
    import torch.nn.functional as F
    from dew_b200.utils.parity import assert_on_par

    def norm_inputs(seed):
        g = torch.Generator(device=DEV).manual_seed(seed)
        return (torch.randn(512, 1024, device=DEV, generator=g).to(torch.bfloat16), (1 + 0.1 * torch.randn(1024, device=DEV, generator=g)).to(torch.bfloat16),
                torch.randn(512, 1024, device=DEV, generator=g).to(torch.bfloat16))

    def norm_arm(fn, dtype):
        def run(seed):
            x, w, dy = norm_inputs(seed)
            x, w = x.to(dtype).requires_grad_(), w.to(dtype).requires_grad_()
            y = fn(x, w)
            y.backward(dy.to(y.dtype))
            return {"y": y, "dx": x.grad, "dw": w.grad}
        return run
    plain = lambda x, w: (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(x.dtype)
    exact = lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert_on_par(norm_arm(lambda x, w: ops.rms_norm(x, w, 1e-6), torch.bfloat16), norm_arm(plain, torch.bfloat16), norm_arm(exact, torch.float64))

    def attn_inputs(seed):
        g = torch.Generator(device=DEV).manual_seed(100 + seed)
        mk = lambda h: torch.randn(1, 512, h, 128, device=DEV, generator=g).to(torch.bfloat16)
        return mk(4), mk(2), mk(2), mk(4)

    def attn_arm(kind):
        def run(seed):
            q, k, v, do = attn_inputs(seed)
            if kind == "truth":
                q, k, v = (t.double().requires_grad_() for t in (q, k, v))
                kk, vv = (t.repeat_interleave(2, 2) for t in (k, v))
                sc = torch.einsum("bshd,bthd->bhst", q, kk) / math.sqrt(128)
                sc = sc.masked_fill(~torch.tril(torch.ones(512, 512, dtype=torch.bool, device=DEV)), float("-inf"))
                o = torch.einsum("bhst,bthd->bshd", torch.softmax(sc, -1), vv)
            else:
                q, k, v = (t.requires_grad_() for t in (q, k, v))
                o = ops.attention(q, k, v, causal=True, kernel="sm100_flash" if kind == "kernel" else "sdpa")
            o.backward(do.to(o.dtype))
            return {"o": o, "dq": q.grad, "dk": k.grad, "dv": v.grad}
        return run
    assert_on_par(attn_arm("kernel"), attn_arm("sdpa"), attn_arm("truth"))
    L.check_status()


def test_atomics_free_kernels_are_bitwise_repeatable():
    """Run-twice determinism (the stand-in for a race detector here): kernels that promise no atomics must return the same
    bits on the same inputs - a missing barrier or a buffer reused too early shows up as a difference."""
    from dew_b200.ops import scan
    from dew_b200.parallel.ep import TokenExchange
    torch.manual_seed(5)

    def twice(fn):
        a = fn()
        torch.cuda.synchronize()
        b = fn()
        torch.cuda.synchronize()
        for x, y in zip(a, b):
            assert torch.equal(x, y)

    # flash attention forward and backward (dQ, dK, dV without atomics)
    qkv = torch.randn(2, 1024, 4 + 2 * 2, 128, device=DEV).to(torch.bfloat16)
    do = torch.randn(2, 1024, 4, 128, device=DEV).to(torch.bfloat16)

    def attn():
        x = qkv.clone().requires_grad_()
        o = ops.attention(x[:, :, :4], x[:, :, 4:6], x[:, :, 6:], causal=True, kernel="sm100_flash")
        o.backward(do)
        return o.detach(), x.grad
    twice(attn)
    # gated delta rule forward + backward
    q, k, v, g, beta, _ = _gdn_inputs(1, 512, 2, 77, False)

    def gdn():
        leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)]
        o, S = scan.chunk_gated_delta_rule(*leaves)
        torch.autograd.backward((o, S), (torch.ones_like(o), torch.ones_like(S) * 0.1))
        return (o.detach(), S.detach(), *[t.grad for t in leaves])
    twice(gdn)
    # MoE exchange: plan, dispatch, combine
    x = torch.randn(512, 256, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(16, device=DEV)[:4] for _ in range(512)])
    w = torch.rand(512, 4, device=DEV)
    ex = TokenExchange(16, "self")

    def moe():
        plan = ex.plan(ids, 256)
        rows = ex.push(x, plan)
        out = ex.pull(rows, plan, w)
        return rows, (out[0] if isinstance(out, tuple) else out)
    twice(moe)
    # CTA-pair GEMM with fp32 accumulation into an existing buffer
    A, Bm = torch.randn(1024, 512, device=DEV).to(torch.bfloat16), torch.randn(1024, 768, device=DEV).to(torch.bfloat16)
    base = torch.randn(512, 768, device=DEV)

    def wgrad():
        out = base.clone()
        ops.gemm(A, Bm, a_mn=True, b_mn=True, out=out, accumulate=True, kernel="sm100_pair")
        return (out,)
    twice(wgrad)
    L.check_status()


def test_bounded_device_wait_runs_out_and_the_context_stays_usable():
    """A wait on a flag that nothing sets gives up after its limit (50 ms here), the kernel returns, the host reads the code
    through the status word as a ``KernelError``, and after the status is cleared the same context runs a GEMM."""
    import ctypes
    import time
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)            # two "ranks": slot 3, nobody ever writes sequence 7
    lib = L.load()
    t0 = time.perf_counter()
    L.check(lib.dewb_wait_flags(L.ptr(flags), ctypes.c_int(3), ctypes.c_int(2), ctypes.c_uint(7), ctypes.c_ulonglong(50_000_000),
                                L.ptr(L.status()), L.stream_ptr()), "wait_flags")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                               # the wait ended by itself
    with pytest.raises(L.KernelError, match="peer"):
        L.check_status()
    L.check_status()                                                    # cleared by the raise above
    a = torch.randn(256, 128, device=DEV).to(torch.bfloat16)
    b = torch.randn(512, 128, device=DEV).to(torch.bfloat16)
    out = ops.gemm(a, b, kernel="sm100_tcgen05")
    assert rel_err(out, a.float() @ b.float().t()) < 1e-2
    # a poisoned status makes later launches return at once instead of waiting again
    L.check(lib.dewb_wait_flags(L.ptr(flags), ctypes.c_int(3), ctypes.c_int(2), ctypes.c_uint(7), ctypes.c_ulonglong(50_000_000),
                                L.ptr(L.status()), L.stream_ptr()), "wait_flags")
    t1 = time.perf_counter()
    L.check(lib.dewb_wait_flags(L.ptr(flags), ctypes.c_int(3), ctypes.c_int(2), ctypes.c_uint(7), ctypes.c_ulonglong(2_000_000_000),
                                L.ptr(L.status()), L.stream_ptr()), "wait_flags")
    torch.cuda.synchronize()
    assert time.perf_counter() - t1 < 1.0
    with pytest.raises(L.KernelError):
        L.check_status()


def test_flash_forward_backward_at_the_training_shape():
    """2 x 4096 tokens, 32 query / 8 kv heads of 128, causal - the shape the dense configuration trains at - against the fp32
    reference computed head group by head group (the full fp32 score tensor would be 4 GB)."""
    torch.manual_seed(11)
    B, S, Hq, Hkv, D = 2, 4096, 32, 8, 128
    qkv = (torch.randn(B, S, Hq + 2 * Hkv, D, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    out = ops.attention(q, k, v, causal=True, kernel="sm100_flash")
    do = torch.randn_like(out)
    out.backward(do)
    got = qkv.grad
    G = Hq // Hkv
    worst = {}
    for h in range(Hkv):                                   # one kv head and its 4 query heads at a time, batch by batch
        for b in range(B):
            rq = qkv.detach()[b:b + 1, :, h * G:(h + 1) * G].float().requires_grad_()
            rk = qkv.detach()[b:b + 1, :, Hq + h:Hq + h + 1].float().requires_grad_()
            rv = qkv.detach()[b:b + 1, :, Hq + Hkv + h:Hq + Hkv + h + 1].float().requires_grad_()
            ref = ops.attention_reference(rq, rk, rv, causal=True)
            ref.backward(do[b:b + 1, :, h * G:(h + 1) * G].float())
            pairs = {"o": (out[b:b + 1, :, h * G:(h + 1) * G], ref), "dq": (got[b:b + 1, :, h * G:(h + 1) * G], rq.grad),
                     "dk": (got[b:b + 1, :, Hq + h:Hq + h + 1], rk.grad), "dv": (got[b:b + 1, :, Hq + Hkv + h:Hq + Hkv + h + 1], rv.grad)}
            for name, (a, r) in pairs.items():
                e = rel_err(a, r) / max(bf16_floor(r), 1e-6)
                worst[name] = max(worst.get(name, 0.0), e)
    # within a small multiple of the rounding floor of a bf16 result (probabilities and dS are rounded to bf16 on the way)
    assert worst["o"] <= 3.0 and worst["dv"] <= 4.0 and worst["dq"] <= 6.0 and worst["dk"] <= 6.0, worst


def test_gemm_ce_gdn_and_grouped_gemm_are_on_par_with_pytorch_bf16_against_float64():
    """The accuracy contract for the remaining tensor-core kernels: over 8 seeds each one's error from a float64 truth stays
    within 1.5x the error of the same op done by PyTorch in bf16 (worst row within 4x)."""
    from dew_b200.ops import grouped as G
    from dew_b200.ops import scan
    from dew_b200.utils.parity import assert_on_par

    # dense GEMM (forward / both gradients through ops.linear)
    def lin_inputs(seed):
        g = torch.Generator(device=DEV).manual_seed(seed)
        return (torch.randn(512, 1024, device=DEV, generator=g).to(torch.bfloat16),
                (torch.randn(768, 1024, device=DEV, generator=g) / 32).to(torch.bfloat16),
                torch.randn(512, 768, device=DEV, generator=g).to(torch.bfloat16))

    def lin_arm(kind):
        def run(seed):
            x, w, dy = lin_inputs(seed)
            dt = torch.float64 if kind == "truth" else torch.bfloat16
            x, w = x.to(dt).requires_grad_(), w.to(dt).requires_grad_()
            y = ops.linear(x, w) if kind == "kernel" else torch.nn.functional.linear(x, w)
            y.backward(dy.to(dt))
            return {"y": y, "dx": x.grad, "dw": w.grad}
        return run
    assert_on_par(lin_arm("kernel"), lin_arm("torch"), lin_arm("truth"))

    # fused linear + cross entropy
    def ce_inputs(seed):
        g = torch.Generator(device=DEV).manual_seed(50 + seed)
        return (torch.randn(384, 256, device=DEV, generator=g).to(torch.bfloat16),
                (torch.randn(4096, 256, device=DEV, generator=g) / 16).to(torch.bfloat16),
                torch.randint(0, 4096, (384,), device=DEV, generator=g))

    def ce_arm(kind):
        def run(seed):
            h, w, tg = ce_inputs(seed)
            dt = torch.float64 if kind == "truth" else torch.bfloat16
            h, w = h.to(dt).requires_grad_(), w.to(dt).requires_grad_()
            if kind == "kernel":
                total, mass = ops.linear_cross_entropy(h, w, tg, chunk=128)
                loss = total / mass
            else:
                logits = torch.nn.functional.linear(h, w)
                loss = torch.nn.functional.cross_entropy(logits.float() if kind == "torch" else logits, tg)
            loss.backward()
            return {"loss": loss.reshape(1), "dh": h.grad, "dw": w.grad}
        return run
    assert_on_par(ce_arm("kernel"), ce_arm("torch"), ce_arm("truth"))

    # grouped (expert) GEMM
    def gmm_arm(kind):
        def run(seed):
            g = torch.Generator(device=DEV).manual_seed(90 + seed)
            T, k, E, d, F_ = 512, 2, 8, 256, 128
            ids = torch.randint(0, E, (T, k), device=DEV, generator=g)
            layout = G.group_layout(ids, E)
            x = torch.randn(T, d, device=DEV, generator=g).to(torch.bfloat16)
            w = (torch.randn(E, F_, d, device=DEV, generator=g) / 16).to(torch.bfloat16)
            xs = G.permute(x, layout, k)
            used = torch.zeros(layout.rows, dtype=torch.bool, device=DEV)
            used[layout.positions] = True
            if kind == "kernel":
                y = G.grouped_linear(xs, w, layout)
            elif kind == "torch":
                y = G._gmm_reference(xs, w, layout, False)                  # fp32 products, rounded to bf16 once
            else:
                y = G._gmm_reference(xs.double(), w.double(), layout, False)
            return {"y": y[used]}
        return run
    assert_on_par(gmm_arm("kernel"), gmm_arm("torch"), gmm_arm("truth"))

    # gated delta rule: kernel against the chunked PyTorch form in bf16, truth = the same form in float64
    def gdn_arm(kind):
        def run(seed):
            q, k, v, gg, beta, _ = _gdn_inputs(1, 256, 2, 300 + seed, False)
            if kind == "kernel":
                o, S = scan.chunk_gated_delta_rule(q, k, v, gg, beta)
            elif kind == "torch":
                with torch.autocast("cuda", dtype=torch.bfloat16):            # the chunk products in bf16, as PyTorch would run them
                    o, S = scan.gated_delta_rule_chunked(q, k, v, gg, beta)
            else:
                o, S = scan.gated_delta_rule_chunked(q.double(), k.double(), v.double(), gg.double(), beta.double())
            return {"o": o, "S": S.float() if kind != "truth" else S}
        return run
    assert_on_par(gdn_arm("kernel"), gdn_arm("torch"), gdn_arm("truth"))


@pytest.mark.parametrize("variant", ["window", "softcap", "sinks", "segments", "window+softcap+sinks", "segments+padding", "full_window"])
def test_flash_variants_forward_backward_on_the_sm100_kernels(variant):
    """Sliding window, soft-capping, attention sinks and packed documents run on the tcgen05 flash kernels (no eager path):
    outputs and every gradient against the fp32 reference of the same variant."""
    torch.manual_seed(hash(variant) % 1000)
    B, S, Hq, Hkv, D = 2, 512, 4, 2, 128
    causal = variant != "full_window"
    q, k, v = (torch.randn(B, S, h, D, device=DEV).to(torch.bfloat16).requires_grad_() for h in (Hq, Hkv, Hkv))
    kw = {}
    sinks = None
    if "window" in variant:
        kw["window"] = 200
    if "softcap" in variant:
        kw["softcap"] = 20.0
    if "sinks" in variant:
        sinks = torch.randn(Hq, device=DEV).requires_grad_()
        kw["sinks"] = sinks
    if "segments" in variant:
        seg = torch.ones(B, S, dtype=torch.int32, device=DEV)
        seg[0, 100:333] = 2
        seg[0, 333:] = 3
        seg[1, 256:] = 2
        if "padding" in variant:
            seg[0, 470:] = 0                                  # padding after the last document
            seg[1, 300:] = 0
        kw["segment_ids"] = seg
    out = ops.attention(q, k, v, causal=causal, kernel="sm100_flash", **kw)
    do = torch.randn_like(out)
    out.backward(do)
    got = [q.grad.clone(), k.grad.clone(), v.grad.clone()] + ([sinks.grad.clone()] if sinks is not None else [])
    rq, rk, rv = (t.detach().float().requires_grad_() for t in (q, k, v))
    rkw = dict(kw)
    if sinks is not None:
        rs = sinks.detach().clone().requires_grad_()
        rkw["sinks"] = rs
    ref = ops.attention_reference(rq, rk, rv, causal=causal, **rkw)
    ref.backward(do.float())
    want = [rq.grad, rk.grad, rv.grad] + ([rs.grad] if sinks is not None else [])
    live = torch.ones(B, S, dtype=torch.bool, device=DEV)
    if "padding" in variant:
        live = kw["segment_ids"] != 0                      # padded rows attend to padding only; nothing reads them
    assert rel_err(out[live], ref[live]) <= 3 * bf16_floor(ref[live]) + 2e-3, rel_err(out[live], ref[live])
    for name, g, r in zip(("dq", "dk", "dv", "dsinks"), got, want):
        assert rel_err(g, r) <= 3 * bf16_floor(r) + 1.5e-2, (name, rel_err(g, r))
    # the selector no longer sends any variant to the eager path on a GPU
    from dew_b200.ops import attn as A
    case = dict(dtype=torch.bfloat16, D=D, S=S, T=S, Hq=Hq, Hkv=Hkv, sinks=sinks is not None, softcap=bool(kw.get("softcap")),
                window=kw.get("window"), segments="segment_ids" in kw, causal=causal, grad=True, unit_d=True)
    assert A._ATTN.select(case) == "sm100_flash"


@pytest.mark.parametrize("M,N,K", [(128, 192, 128), (256, 384, 256), (1000, 2816, 2048), (4096, 2048, 1408 - 1408 % 128)])
def test_mxfp8_block_scaled_gemm(M, N, K):
    """tcgen05 kind::mxf8f6f4.block_scale: the quantiser equals the PyTorch restatement bit for bit, and the product equals the
    fp32 product of the de-quantised operands (the tensor core applies the 1 x 32 block scales itself)."""
    from dew_b200.ops import mx
    torch.manual_seed(M + N)
    # blocks of very different magnitude within a row, so that a wrong scale factor cannot hide
    mag = torch.exp2(torch.randint(-6, 7, (M, K // 32), device=DEV).float()).repeat_interleave(32, 1)
    a = (torch.randn(M, K, device=DEV) * mag).to(torch.bfloat16)
    magb = torch.exp2(torch.randint(-5, 6, (N, K // 32), device=DEV).float()).repeat_interleave(32, 1)
    b = (torch.randn(N, K, device=DEV) * magb / math.sqrt(K)).to(torch.bfloat16)
    aq, sa = mx.quantize_mx(a)
    bq, sb = mx.quantize_mx(b, sf_rows=(N + 192 + 127) // 128 * 128)
    rq, re = mx.quantize_mx_reference(a)
    assert torch.equal(aq.view(torch.uint8), rq.view(torch.uint8))
    assert torch.equal(mx.unpack_scales(sa, M, K), re)
    out = mx.gemm_mx(aq, sa, bq, sb)
    ref = mx.dequantize_mx(aq, mx.unpack_scales(sa, M, K)) @ mx.dequantize_mx(bq, mx.unpack_scales(sb, N, K)).t()
    assert rel_err(out, ref) <= 2 * bf16_floor(ref) + 1e-3, rel_err(out, ref)
    # and the quantisation itself costs what 1 x 32 e4m3 blocks cost against the bf16 product
    exact = a.float() @ b.float().t()
    assert rel_err(out, exact) < 6e-2


def test_mxfp8_grouped_linear_forward_backward():
    """Expert projection in MXFP8 (forward and input gradient on the block-scaled kernel, weight gradient in bf16) against the
    bf16 grouped GEMM."""
    from dew_b200.ops import grouped as G
    from dew_b200.ops import mx
    torch.manual_seed(3)
    T, k, E, d, F_ = 1000, 2, 8, 256, 384
    ids = torch.randint(0, E, (T, k), device=DEV)
    ids[ids == 5] = 4                                       # one empty expert
    layout = G.group_layout(ids, E)
    xs = G.permute(torch.randn(T, d, device=DEV).to(torch.bfloat16), layout, k)
    used = torch.zeros(layout.rows, dtype=torch.bool, device=DEV)
    used[layout.positions] = True
    w = (torch.randn(E, F_, d, device=DEV) / math.sqrt(d)).to(torch.bfloat16)
    a, b = xs.clone().requires_grad_(), w.clone().requires_grad_()
    y = mx.mx_grouped_linear(a, b, layout)
    dy = torch.randn_like(y) * used[:, None]
    y.backward(dy)
    ra, rb = xs.clone().requires_grad_(), w.clone().requires_grad_()
    ry = G.grouped_linear(ra, rb, layout)
    ry.backward(dy)
    assert rel_err(y[used], ry[used]) < 6e-2
    assert rel_err(a.grad[used], ra.grad[used]) < 6e-2
    assert rel_err(b.grad, rb.grad) < 1e-2                  # the weight gradient runs the bf16 kernel in both
    assert torch.all(y[~used] == 0)


def test_fused_decode_step_from_the_packed_projection():
    """Rotation + cache append in one kernel and paged attention reading the queries in place equal the unfused path
    (rope kernel, append kernel, contiguous slices, attention) bit for bit, and a -1 position leaves its row alone."""
    from dew_b200.nn.kv_cache import KVCache, KVStore
    torch.manual_seed(21)
    rows, max_len, Hq, Hkv, D = 6, 700, 8, 2, 128

    def filled():
        torch.manual_seed(22)
        store = KVStore(KVCache(page_size=64), 1, rows, max_len, Hkv, D, torch.bfloat16, DEV)
        perm = torch.randperm(store.pages, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1)).to(torch.int32)
        store.page_table.copy_(perm.reshape(rows, store.max_pages))
        lengths = torch.tensor([1, 17, 256, 511, 640, 300], device=DEV)
        S = int(lengths.max())
        k = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
        v = torch.randn(rows, S, Hkv, D, device=DEV).to(torch.bfloat16)
        pos = torch.arange(S, device=DEV)[None].expand(rows, S).clone()
        pos[pos >= lengths[:, None]] = -1
        store.write(0, k, v, pos)
        return store, lengths
    cos, sin = ops.rope_tables(1024, D, 10000.0, torch.device(DEV))
    qkv = torch.randn(rows, Hq + 2 * Hkv, D, device=DEV).to(torch.bfloat16)
    a, lengths = filled()
    positions = lengths.clone()
    positions[5] = -1                                              # an idle row
    fused_in = qkv.clone()
    assert a.can_decode_packed(fused_in, Hq)
    fused = a.decode_packed(0, fused_in, cos, sin, positions, Hq)
    b, _ = filled()
    rot = ops.rope(qkv.clone()[:, None], cos, sin, positions.clamp_min(0)[:, None], rot_heads=Hq + Hkv)[:, 0]
    q, k, v = rot[:, :Hq], rot[:, Hq:Hq + Hkv], rot[:, Hq + Hkv:]
    plain = b.attend(0, q[:, None], k[:, None], v[:, None], positions[:, None])[:, 0]
    live = positions >= 0
    assert torch.equal(fused_in[5], qkv[5])                        # the idle row's projection was not rotated
    assert torch.equal(fused_in[live][:, :Hq + Hkv], rot[live][:, :Hq + Hkv]), "rotation differs"
    # (the page past the addressable pool only collects the writes of padding positions, in no particular order)
    assert torch.equal(a.v[0, :a.pages], b.v[0, :b.pages]), "value cache differs"
    assert torch.equal(a.k[0, :a.pages], b.k[0, :b.pages]), "key cache differs"
    assert torch.equal(fused[live], plain[live]), float((fused[live].float() - plain[live].float()).abs().max())


@pytest.mark.parametrize("M,N,K", [(128, 768, 4096), (128, 4096, 512), (128, 4096, 1792), (1, 768, 4096), (7, 200, 520), (100, 16032, 4096),
                                   (128, 128, 64), (33, 3584, 4096)])
@pytest.mark.parametrize("pdl", [1, 0])
def test_weight_streaming_gemm_for_decode(M, N, K, pdl, monkeypatch):
    """The decode-sized product (at most 128 rows): tcgen05 tiles with K split over a thread-block cluster and summed through
    distributed shared memory, against the fp32 product; launched with and without programmatic dependent launch; twice, the
    same bits."""
    from dew_b200.ops import functional as Fn
    monkeypatch.setattr(Fn, "_SKINNY_PDL", pdl)
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    before = dict(Fn._GEMM.routes.get("sm100_skinny", {"calls": 0}))["calls"]
    y = ops.gemm(x, w, kernel="sm100_skinny")
    assert Fn._GEMM.routes["sm100_skinny"]["calls"] == before + 1          # the kernel under test took the call
    assert rel_err(y, ref) <= 6e-3, rel_err(y, ref)
    assert torch.equal(ops.gemm(x, w, kernel="sm100_skinny"), y)
    # a strided activation view (rows of a wider tensor), as the decode step passes
    wide = torch.randn(M, K + 64, device=DEV).to(torch.bfloat16)
    assert rel_err(ops.gemm(wide[:, :K], w, kernel="sm100_skinny"), wide[:, :K].float() @ w.float().t()) <= 6e-3
    L.check_status()


@pytest.mark.parametrize("M,F,K", [(128, 1792, 4096), (128, 14336, 4096), (5, 64, 128), (77, 448, 1000)])
def test_gate_up_projection_with_swiglu_in_the_epilogue(M, F, K):
    """silu(x Wg^T) * (x Wu^T) as one kernel (the activation in the weight-streaming GEMM's epilogue) against the two-step fp32
    computation, and through the MLP module without autograd."""
    torch.manual_seed(F)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device=DEV) * 0.03).to(torch.bfloat16)
    with torch.no_grad():
        y = ops.linear_swiglu(x, w, fused=True)
    gu = x.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    assert y.shape == (M, F) and rel_err(y, ref) <= 8e-3, rel_err(y, ref)
    with torch.no_grad():
        assert torch.equal(ops.linear_swiglu(x, w, fused=True), y)
    # with autograd the two-step path runs and agrees
    xg = x.clone().requires_grad_()
    y2 = ops.linear_swiglu(xg, w)
    assert rel_err(y2, ref) <= 8e-3
    L.check_status()


@pytest.mark.parametrize("kernel", ["sm100_tcgen05", "sm100_pair"])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 1024), (1000, 1160, 264)])
def test_gemm_bias_in_the_epilogue(kernel, M, N, K):
    """D = A B^T + bias with the bias row added by the product's epilogue (both dense kernels), and through the Linear autograd
    node (forward value, bias gradient)."""
    torch.manual_seed(M)
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    b = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    y = ops.gemm(a, b, bias=bias, kernel=kernel)
    assert rel_err(y, ref) <= 6e-3, rel_err(y, ref)
    assert rel_err(ops.gemm(a, b, bias=bias, kernel=kernel, alpha=0.5), 0.5 * (a.float() @ b.float().t()) + bias.float()) <= 6e-3
    xa = a.clone().requires_grad_()
    bp = bias.clone().requires_grad_()
    out = ops.linear(xa, b, bp)
    assert rel_err(out, ref) <= 6e-3
    out.float().sum().backward()
    assert rel_err(bp.grad, torch.full_like(bias, float(M))) <= 1e-2
    L.check_status()
