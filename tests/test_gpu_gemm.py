"""tcgen05 GEMM against an fp32 PyTorch matmul of the same bf16 operands."""
import pytest
import torch

from solarwm_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(a, b, layout):
    af, bf = a.float(), b.float()
    if layout == ops.NT:
        return af @ bf.t()
    if layout == ops.NN:
        return af @ bf
    return af.t() @ bf


def _operands(M, N, K, layout, gen):
    dev = "cuda"
    mk = lambda *s: (torch.randn(*s, generator=gen, device=dev) * 0.5).to(torch.bfloat16)
    if layout == ops.NT:
        return mk(M, K), mk(N, K)
    if layout == ops.NN:
        return mk(M, K), mk(K, N)
    return mk(K, M), mk(K, N)


def _check(c, ref, K):
    err = (c.float() - ref).abs().max().item()
    tol = 0.02 * (K ** 0.5) * 0.25 + 0.05
    assert err <= tol, f"max abs err {err} > {tol}"
    # relative Frobenius error is the tight check (bf16 output rounding ~ 2^-9)
    rel = ((c.float() - ref).norm() / ref.norm().clamp_min(1e-6)).item()
    assert rel < 4e-3, f"relative error {rel}"


@pytest.mark.parametrize("layout", [ops.NT, ops.NN, ops.TN])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (320, 384, 128), (1000, 776, 200),
                                   (4096, 3072, 3072), (31, 1536, 256)])  # noqa: E501
def test_gemm_layouts(layout, shape):
    M, N, K = shape
    if layout == ops.TN and M % 8 != 0:
        pytest.skip("TN stores A as [K, M]: M must keep rows 16-byte aligned")
    gen = torch.Generator(device="cuda").manual_seed(M + N + K + layout)
    a, b = _operands(M, N, K, layout, gen)
    c = ops.gemm(a, b, layout)
    ops.check_status()
    _check(c, _ref(a, b, layout), K)


def test_gemm_bias_gelu_fp32_accumulate():
    gen = torch.Generator(device="cuda").manual_seed(7)
    M, N, K = 520, 640, 320
    a, b = _operands(M, N, K, ops.NT, gen)
    bias = torch.randn(N, generator=gen, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float()
    c = ops.gemm(a, b, ops.NT, bias=bias)
    _check(c, ref, K)
    c = ops.gemm(a, b, ops.NT, bias=bias, act="gelu")
    _check(c, torch.nn.functional.gelu(ref, approximate="tanh"), K)
    c32 = ops.gemm(a, b, ops.NT, out_dtype=torch.float32)
    assert c32.dtype == torch.float32
    assert ((c32 - (ref - bias.float())).norm() / ref.norm()).item() < 1e-4
    acc = torch.full((M, N), 1.5, dtype=torch.float32, device="cuda")
    ops.gemm(a, b, ops.NT, out=acc, accumulate=True)
    assert ((acc - (ref - bias.float() + 1.5)).norm() / ref.norm()).item() < 1e-4
    ops.check_status()


def test_gemm_strided_operands_and_output():
    gen = torch.Generator(device="cuda").manual_seed(11)
    big = (torch.randn(300, 3 * 256, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(128, 256, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    a = big[:, 256:512]                      # row stride 768
    c = ops.gemm(a, w, ops.NT)
    _check(c, a.float() @ w.float().t(), 256)
    out = torch.zeros(300, 512, dtype=torch.bfloat16, device="cuda")
    ops.gemm(a, w, ops.NT, out=out[:, 128:256])
    _check(out[:, 128:256], a.float() @ w.float().t(), 256)
    assert out[:, :128].abs().max().item() == 0 and out[:, 256:].abs().max().item() == 0
    ops.check_status()


def test_linear_autograd_matches_reference():
    gen = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(384, 256, generator=gen, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(512, 256, generator=gen, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(512, generator=gen, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = xr @ wr.t() + br
    yr.backward(g.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (b.grad, br.grad)):
        rel = ((got.float() - ref).norm() / ref.norm()).item()
        assert rel < 6e-3, rel
    assert ops.COUNTERS.get("gemm", 0) >= 3


@pytest.mark.parametrize("layout", [ops.NT, ops.NN, ops.TN])
@pytest.mark.parametrize("shape", [(256, 256, 64), (300, 520, 192), (1000, 776, 200), (4096, 3072, 1024)])
def test_cta_pair_kernel_is_bit_identical_to_single_cta(layout, shape):
    """The cta_group::2 kernel (256-row tiles over two SMs) against the single-CTA kernel and the fp32 reference,
    including tails in M (the second CTA of the last pair owns no rows) and in N and K."""
    import ctypes

    from solarwm_b200.ops import _lib

    M, N, K = shape
    if layout == ops.TN and M % 8:
        pytest.skip("TN needs a 16-byte aligned row stride of A")
    lib = _lib.load()
    lib.solar_gemm_pair_mode.argtypes = [ctypes.c_int]
    gen = torch.Generator(device="cuda").manual_seed(11)
    a, b = _operands(M, N, K, layout, gen)
    bias = (torch.randn(N, generator=gen, device="cuda") * 0.1).to(torch.bfloat16)
    old = lib.solar_gemm_pair_mode(0)
    try:
        single = ops.gemm(a, b, layout, bias=bias)
        single32 = ops.gemm(a, b, layout, out_dtype=torch.float32)
        lib.solar_gemm_pair_mode(1)
        pair = ops.gemm(a, b, layout, bias=bias)
        pair32 = ops.gemm(a, b, layout, out_dtype=torch.float32)
        acc = pair32.clone()
        ops.gemm(a, b, layout, out=acc, accumulate=True)
    finally:
        lib.solar_gemm_pair_mode(old)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(single, pair) and torch.equal(single32, pair32)
    _check(pair32, _ref(a, b, layout), K)
    assert torch.allclose(acc, 2 * pair32, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("M,F,K,bias", [(300, 192, 256, False), (1000, 256, 128, True), (130, 704, 64, True)])
def test_swiglu_epilogue_matches_fp32_reference(M, F, K, bias):
    """silu(x Wg^T + bg) * (x Wu^T + bu) computed in the GEMM epilogue from block-interleaved weights, on both the
    single-CTA and the CTA-pair kernel."""
    import ctypes

    from solarwm_b200 import ops
    from solarwm_b200.ops import _lib
    from solarwm_b200.ops import functional as F_

    g = torch.Generator(device="cuda").manual_seed(M + F)
    x = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, generator=g, device="cuda") / K ** 0.5).to(torch.bfloat16)
    b = (torch.randn(2 * F, generator=g, device="cuda") * 0.1).to(torch.bfloat16) if bias else None
    xf, wf = x.float(), w.float()
    gate, up = xf @ wf[:F].t(), xf @ wf[F:].t()
    if bias:
        gate, up = gate + b[:F].float(), up + b[F:].float()
    want = torch.nn.functional.silu(gate) * up
    lib = _lib.load()
    lib.solar_gemm_pair_mode.argtypes = [ctypes.c_int]
    for mode in (0, 1):
        old = lib.solar_gemm_pair_mode(mode)
        try:
            got = F_.linear_swiglu(x, F_.interleave_gate_up(w), None if b is None else F_.interleave_gate_up(b))
        finally:
            lib.solar_gemm_pair_mode(old)
        ops.check_status()
        assert got.shape == (M, F)
        err = (got.float() - want).abs().max() / want.abs().max()
        assert err < 2e-2, (mode, float(err))
