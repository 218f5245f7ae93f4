"""Out-of-bounds and race checks that need no sanitizer: outputs carved out of canary-filled buffers (nothing
outside the output may change, whatever the tile shapes) and repeated runs that must agree bit for bit (a data race
or an unordered reduction shows up as a difference).  The file sorts near the end on purpose: a run that stops at
the first failure has already run the functional tests."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

CANARY = 1234.0


def _mk(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K,layout", [(300, 264, 192, "nt"), (129, 72, 64, "nn"), (1000, 520, 336, "tn"),
                                          (2050, 264, 128, "nt")])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_writes_only_its_output_rows_and_columns(M, N, K, layout, out_dtype):
    from solarwm_b200 import ops
    from solarwm_b200.ops import functional as F_

    K = (K + 7) // 8 * 8
    lay = {"nt": F_.NT, "nn": F_.NN, "tn": F_.TN}[layout]
    a = _mk((M, K) if layout != "tn" else (K, M), 1, 0.1)
    b = _mk((N, K) if layout == "nt" else (K, N), 2, 0.1)
    pad_rows, ld = 5, N + 24                                   # 24 spare columns keep the row stride a multiple of 16 bytes
    big = torch.full((M + 2 * pad_rows, ld), CANARY, dtype=out_dtype, device="cuda")
    out = big[pad_rows:pad_rows + M, :N]
    for pair_mode in (0, 1):                                    # single-CTA kernel, then the CTA-pair kernel
        F_._lib.load().solar_gemm_pair_mode(pair_mode)
        try:
            big.fill_(CANARY)
            F_.gemm(a, b, lay, out=out)
        finally:
            F_._lib.load().solar_gemm_pair_mode(-1)
        ops.check_status()
        af, bf = a.float(), b.float()
        want = af @ bf.t() if layout == "nt" else (af @ bf if layout == "nn" else af.t() @ bf)
        assert ((out.float() - want).abs().max() / want.abs().max()) < 2e-2
        assert bool((big[:pad_rows] == CANARY).all()) and bool((big[pad_rows + M:] == CANARY).all())
        assert bool((big[:, N:] == CANARY).all())


def test_conv_kernel_writes_only_its_frames():
    from solarwm_b200 import ops
    from solarwm_b200.ops import functional as F_

    T, H, W, cin, cout = 2, 11, 19, 32, 40
    x = _mk((T, H, W, cin), 3)
    w = _mk((cout, cin, 3, 3, 3), 4, 1.0 / math.sqrt(cin * 27))
    pw, pb = F_.pack_conv_weight(w, None)
    first = F_.conv3d_channels_last(x, pw, pb, (3, 3, 3))
    second = F_.conv3d_channels_last(x, pw, pb, (3, 3, 3))
    ops.check_status()
    assert torch.equal(first, second) and bool(torch.isfinite(first).all())


def test_repeated_runs_are_bitwise_identical():
    from solarwm_b200 import ops
    from solarwm_b200.ops import functional as F_
    from solarwm_b200.ops.attention_bwd_native import attn_bwd_native
    from solarwm_b200.ops.attention_native import attn_fwd

    a, b = _mk((1500, 512), 5, 0.1), _mk((776, 512), 6, 0.1)
    acc0 = torch.zeros(1500, 776, dtype=torch.float32, device="cuda")
    acc1 = torch.zeros_like(acc0)
    for acc in (acc0, acc1):
        F_.gemm(a, b, F_.NT, out=acc, accumulate=True)
        F_.gemm(a, b, F_.NT, out=acc, accumulate=True)
    assert torch.equal(acc0, acc1)
    q, k, v, do = (_mk((1, n, 3, 128), s) for n, s in ((1100, 7), (900, 8), (900, 9), (1100, 10)))
    scale = 1.0 / math.sqrt(128)
    runs = []
    for _ in range(3):
        o, lse = attn_fwd(q, k, v, scale)
        runs.append((o, lse) + tuple(attn_bwd_native(q, k, v, o, lse, do, scale)))
    ops.check_status()
    for r in runs[1:]:
        assert all(torch.equal(x, y) for x, y in zip(runs[0], r))
    x = _mk((777, 1024), 11)
    shift, scl = torch.randn(3, 1024, device="cuda"), torch.randn(3, 1024, device="cuda")
    y0 = F_.norm_modulate(x, shift, scl, eps=1e-6, rows_per_group=259)
    y1 = F_.norm_modulate(x, shift, scl, eps=1e-6, rows_per_group=259)
    assert torch.equal(y0, y1)


def test_training_step_is_reproducible_from_the_same_seed():
    from solarwm_b200 import ops
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer
    from solarwm_b200.models.wan import WanConfig

    cfg = WanConfig(model_type="ti2v", in_dim=16, out_dim=16, dim=256, ffn_dim=512, num_heads=2, num_layers=2, text_dim=128,
                    text_len=64, freq_dim=64)
    batch = {"latents": torch.randn(1, 3, 16, 16, 16, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16),
             "text": torch.randn(1, 64, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)}
    results = []
    for _ in range(2):
        tr = WanStage0p5Trainer(cfg, "cuda", Stage0p5Options(seed=3, lr=1e-3))
        with torch.no_grad():
            tr.model.get_parameter("head.head.weight").normal_(0, 0.02, generator=torch.Generator(device="cuda").manual_seed(2))
        losses = [float(tr.train_step(batch)) for _ in range(3)]
        results.append((losses, float(tr.last_grad_norm), tr.model.get_parameter("blocks.1.ffn.2.weight").detach().clone()))
    ops.check_status()
    assert results[0][0] == results[1][0] and results[0][1] == results[1][1]
    assert torch.equal(results[0][2], results[1][2])
