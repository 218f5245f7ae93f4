"""Per-kernel timing with CUDA events (warm-up, L2 flush between iterations, synchronised on both
sides) and roofline fractions against the measured peaks of the box.

    python -m solarwm_b200.utils.kernel_bench gemm --m 27280 --n 3072 --k 3072 --layout nt
    python -m solarwm_b200.utils.kernel_bench attention --seq 27280 --heads 24 --head-dim 128 [--backward]
    python -m solarwm_b200.utils.kernel_bench rowops --rows 27280 --dim 3072
    python -m solarwm_b200.utils.kernel_bench suite            # the Wan-5B block shapes
    python -m solarwm_b200.utils.kernel_bench probe --family rows|pointwise|headops|zero|attention|attention_bwd|masked_attention|scatter|conv|gemm
                                                               # one launch of every kernel of a family on a case
                                                               # larger than L2 and a few hundred MB at most: the
                                                               # program a counter capture (ncu -k ... -c N) runs

Each line of output is one JSON object: the op, its shape, milliseconds (median of the timed
iterations), achieved TFLOP/s or GB/s, the fraction of the measured peak, and the same numbers
for the library kernel (cuBLAS / SDPA) that the hand-written kernel replaces.
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

from .. import ops

_PEAKS = None


def peaks():
    """Measured copy bandwidth / bf16 GEMM throughput of this pool (fallback: earlier measurement)."""
    global _PEAKS
    if _PEAKS is None:
        p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
        if p.exists():
            d = json.loads(p.read_text())
            _PEAKS = {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
        else:
            _PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}
    return _PEAKS


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _flush.zero_()


def time_fn(fn, iters=10, warmup=3, flush=True):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            flush_l2()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def bench_gemm(M, N, K, layout="nt", out_f32=False, iters=10):
    lay = {"nt": ops.NT, "nn": ops.NN, "tn": ops.TN}[layout]
    dev = "cuda"
    if lay == ops.NT:
        a, b = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
        lib = lambda: torch.matmul(a, b.t())
    elif lay == ops.NN:
        a, b = torch.randn(M, K, device=dev).bfloat16(), torch.randn(K, N, device=dev).bfloat16()
        lib = lambda: torch.matmul(a, b)
    else:
        a, b = torch.randn(K, M, device=dev).bfloat16(), torch.randn(K, N, device=dev).bfloat16()
        lib = lambda: torch.matmul(a.t(), b)
    out = torch.empty(M, N, device=dev, dtype=torch.float32 if out_f32 else torch.bfloat16)
    ms = time_fn(lambda: ops.gemm(a, b, lay, out=out), iters)
    ms_lib = time_fn(lib, iters)
    fl = 2.0 * M * N * K
    pk = peaks()
    return {"op": "gemm", "layout": layout, "M": M, "N": N, "K": K, "out": "f32" if out_f32 else "bf16",
            "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
            "frac_of_peak": round(fl / ms / 1e9 / pk["bf16_tflops"], 3), "peak_src": pk["src"],
            "cublas_ms": round(ms_lib, 4), "cublas_tflops": round(fl / ms_lib / 1e9, 1),
            "speedup_vs_cublas": round(ms_lib / ms, 3)}


def bench_attention(S, H, D, Sk=None, backward=False, iters=5):
    dev = "cuda"
    Sk = Sk or S
    q = torch.randn(1, S, H, D, device=dev).bfloat16().requires_grad_(backward)
    k = torch.randn(1, Sk, H, D, device=dev).bfloat16().requires_grad_(backward)
    v = torch.randn(1, Sk, H, D, device=dev).bfloat16().requires_grad_(backward)
    fl = 4.0 * S * Sk * H * D
    res = {"op": "attention", "S": S, "Sk": Sk, "H": H, "D": D, "backward": backward}
    for name in ("native", "library"):
        try:
            if backward:
                o = ops.attention(q, k, v, backend=name)
                g = torch.randn_like(o)

                def run():
                    q.grad = k.grad = v.grad = None
                    o.backward(g, retain_graph=True)

                ms = time_fn(run, iters)
                f = fl * 2.5
            else:
                with torch.no_grad():
                    ms = time_fn(lambda: ops.attention(q, k, v, backend=name), iters)
                f = fl
            res[f"{name}_ms"] = round(ms, 4)
            res[f"{name}_tflops"] = round(f / ms / 1e9, 1)
            if name == "native":
                res["frac_of_peak"] = round(f / ms / 1e9 / peaks()["bf16_tflops"], 3)
        except Exception as exc:  # noqa: BLE001
            res[f"{name}_error"] = repr(exc)[:200]
    res["peak_src"] = peaks()["src"]
    return res


def bench_rowops(R, D, iters=10):
    dev = "cuda"
    x = torch.randn(R, D, device=dev).bfloat16()
    y = torch.randn(R, D, device=dev).bfloat16()
    G = max(R // 880, 1)
    mod = torch.randn(G + 1, 6, D, device=dev)
    rpg = (R + G - 1) // G
    pk = peaks()
    out = []

    def add(name, fn, bytes_moved):
        ms = time_fn(fn, iters)
        gbs = bytes_moved / ms / 1e6
        out.append({"op": name, "rows": R, "D": D, "ms": round(ms, 4), "gbs": round(gbs, 1),
                    "frac_of_peak": round(gbs / pk["hbm_gbs"], 3), "peak_src": pk["src"]})

    with torch.no_grad():
        add("norm_modulate_fwd", lambda: ops.norm_modulate(x, mod[:, 0], mod[:, 1], rows_per_group=rpg), 2 * R * D * 2)
        add("gated_residual", lambda: ops.gated_residual(x, y, mod[:, 2], rows_per_group=rpg), 3 * R * D * 2)
        w = torch.ones(D, device=dev)
        add("rmsnorm_rope_fwd(no rope)", lambda: ops.rmsnorm_rope(x, w, None), 2 * R * D * 2)
        add("gelu_fwd", lambda: ops.gelu(x), 2 * R * D * 2)
    return out


def bench_conv(T, H, W, cin, cout, kernel=(3, 3, 3), iters=5):
    """Implicit-GEMM causal convolution on channels-last bf16 against torch's convolution (cuDNN) on the same
    problem in its channels_last_3d layout."""
    import torch.nn.functional as F

    from ..ops import functional as F_

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(T, H, W, cin, device="cuda", generator=g).bfloat16()
    w = (torch.randn(cout, cin, *kernel, device="cuda", generator=g) / (cin * 27) ** 0.5).bfloat16()
    b = torch.zeros(cout, device="cuda").bfloat16()
    pw, pb = F_.pack_conv_weight(w, b)
    ms = time_fn(lambda: F_.conv3d_channels_last(x, pw, pb, kernel), iters)
    kt, kh, kw = kernel
    xl = F.pad(x.permute(3, 0, 1, 2).unsqueeze(0), (kw // 2, kw // 2, kh // 2, kh // 2, kt - 1, 0))
    xl = xl.contiguous(memory_format=torch.channels_last_3d)
    wl = w.contiguous(memory_format=torch.channels_last_3d)
    ms_lib = time_fn(lambda: F.conv3d(xl, wl, b), iters)
    fl = 2.0 * T * H * W * cin * cout * kt * kh * kw
    pk = peaks()
    return {"op": "conv3d", "T": T, "H": H, "W": W, "cin": cin, "cout": cout, "kernel": list(kernel),
            "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
            "frac_of_peak": round(fl / ms / 1e9 / pk["bf16_tflops"], 3), "peak_src": pk["src"],
            "cudnn_ms": round(ms_lib, 4), "speedup_vs_cudnn": round(ms_lib / ms, 3)}


def probe(family: str, rows: int = 27280, dim: int = 3072) -> dict:
    """Launch every kernel of ``family`` once (after one warm-up launch of each) on inputs that exceed the L2 but stay
    within a few hundred MB, and return {kernel: algorithmic bytes or FLOPs per launch}: the denominators for the
    HBM-bytes-vs-algorithmic-bytes line of a counter summary."""
    import math

    from ..ops import functional as F_

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)          # noqa: E731
    R, D = rows, dim
    plan = {}

    def run(name, fn, algorithmic):
        fn()                                   # warm-up (first-use attributes, allocator)
        torch.cuda.synchronize()
        flush_l2()
        fn()
        torch.cuda.synchronize()
        plan[name] = algorithmic

    if family == "rows":
        x, y = rnd(R, D).bfloat16(), rnd(R, D).bfloat16()
        G = max(R // 880, 1)
        rpg = (R + G - 1) // G
        mod = rnd(G + 1, 6, D)
        w = torch.ones(D, device=dev)
        rope = torch.stack([torch.cos(rnd(R, 64)), torch.sin(rnd(R, 64))], -1).contiguous()
        xr = x.clone().requires_grad_(True)
        sh, sc, gt = (mod[:, i].clone().requires_grad_(True) for i in range(3))
        with torch.no_grad():
            run("norm_modulate_fwd", lambda: ops.norm_modulate(x, mod[:, 0], mod[:, 1], rows_per_group=rpg), {"bytes": 4 * R * D})
            run("gated_residual", lambda: ops.gated_residual(x, y, mod[:, 2], rows_per_group=rpg), {"bytes": 6 * R * D})
            run("rmsnorm_rope_fwd", lambda: ops.rmsnorm_rope(x, w, rope), {"bytes": 4 * R * D + 8 * R * 64})
        out = ops.norm_modulate(xr, sh, sc, rows_per_group=rpg)
        run("norm_modulate_bwd+colreduce", lambda: torch.autograd.grad(out, (xr, sh, sc), y, retain_graph=True),
            {"bytes": 6 * R * D + 4 * R * D})
        out2 = ops.gated_residual(xr, y, gt, rows_per_group=rpg)
        run("gated_residual_bwd+colreduce", lambda: torch.autograd.grad(out2, (xr, gt), y, retain_graph=True), {"bytes": 8 * R * D})
        wr = w.clone().requires_grad_(True)
        out3 = ops.rmsnorm_rope(xr, wr, rope)
        run("rmsnorm_rope_bwd+dw", lambda: torch.autograd.grad(out3, (xr, wr), y, retain_graph=True), {"bytes": 10 * R * D})
    elif family == "pointwise":
        n = R * D
        x, y = rnd(R, D).bfloat16(), rnd(R, D).bfloat16()
        xr = x.clone().requires_grad_(True)
        with torch.no_grad():
            run("gelu_fwd", lambda: ops.gelu(x), {"bytes": 4 * n})
        o = ops.gelu(xr)
        run("gelu_bwd", lambda: torch.autograd.grad(o, xr, y, retain_graph=True), {"bytes": 6 * n})
        F = 31
        lat, noise = rnd(F, 48, 44, 80).bfloat16(), rnd(F, 48, 44, 80).bfloat16()
        sig = torch.rand(F, device=dev)
        run("flow(add_noise)", lambda: ops.add_noise(lat, noise, sig), {"bytes": 8 * lat.numel()})
        run("mse_fwd", lambda: ops.weighted_masked_mse(lat, noise, torch.ones(F, device=dev), torch.ones(F, device=dev)),
            {"bytes": 4 * lat.numel()})
        m = 64 * 1024 * 1024
        master, m1, m2, gr = (torch.zeros(m, device=dev) for _ in range(4))
        live = torch.zeros(m, device=dev, dtype=torch.bfloat16)
        scale, skip = torch.ones(1, device=dev), torch.zeros(1, device=dev, dtype=torch.int32)
        run("adamw", lambda: ops.adamw_(master, m1, m2, gr, live=live, lr=1e-4, beta1=0.9, beta2=0.99, eps=1e-8, wd=0.01,
                                        step=1, grad_scale=scale, skip=skip), {"bytes": m * (4 * 4 + 3 * 4 + 2)})
        run("sumsq", lambda: ops.sumsq(gr), {"bytes": 4 * m})
        frame = rnd(3, 768, 1344).bfloat16()
        run("rgb8", lambda: ops.rgb8(frame), {"bytes": frame.numel() * 3})
    elif family == "headops":
        H = D // 128
        x = rnd(R, D).bfloat16()
        w = torch.ones(128, device=dev)
        cos, sin = torch.cos(rnd(R, 96)).contiguous(), torch.sin(rnd(R, 96)).contiguous()
        mats = torch.eye(4, device=dev).repeat(R, 1, 1).contiguous()
        with torch.no_grad():
            run("headop_fwd", lambda: ops.head_norm_rope_prope(x, w, cos, sin, mats, heads=H), {"bytes": 4 * R * D + R * (96 * 8 + 64)})
    elif family == "zero":
        import ctypes

        from ..ops._lib import load, ptr, stream_handle

        lib = load()
        n = 64 * 1024 * 1024
        grads = torch.randn(n, device=dev)
        out, ssq = torch.empty(n, device=dev), torch.zeros(1, device=dev)
        one = (ctypes.c_void_p * 1)(grads.data_ptr())
        run("zero_reduce(1 rank)", lambda: lib.solar_zero_reduce(one, ctypes.c_int(1), ctypes.c_longlong(0), ctypes.c_longlong(n),
                                                                ptr(out), ptr(ssq), ctypes.c_int(0), stream_handle()),
            {"bytes": 8 * n})
        params = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        master, m1, m2 = (torch.zeros(n, device=dev) for _ in range(3))
        scale, skip = torch.ones(1, device=dev), torch.zeros(1, device=dev, dtype=torch.int32)
        pp = (ctypes.c_void_p * 1)(params.data_ptr())
        run("zero_adamw_push(1 rank)", lambda: lib.solar_zero_adamw_push(
            pp, ctypes.c_int(1), ctypes.c_int(1), ctypes.c_longlong(0), ctypes.c_longlong(n), ptr(master), ptr(m1), ptr(m2),
            ptr(out), None, ctypes.c_float(1e-4), ctypes.c_float(0.9), ctypes.c_float(0.99), ctypes.c_float(1e-8),
            ctypes.c_float(0.01), ctypes.c_int(1), ctypes.c_float(0.0), ptr(scale), ptr(skip), ctypes.c_int(0),
            stream_handle()), {"bytes": n * (4 * 4 + 3 * 4 + 2)})
    elif family in ("attention", "attention_bwd"):
        from ..ops.attention_bwd_native import attn_bwd_native
        from ..ops.attention_native import attn_fwd

        S, H, Dh = 16384, 12, 128
        q, k, v = (rnd(1, S, H, Dh).bfloat16() for _ in range(3))
        scale = 1.0 / math.sqrt(Dh)
        fl = 4.0 * S * S * H * Dh
        if family == "attention":
            run("attn_fwd", lambda: attn_fwd(q, k, v, scale), {"flops": fl, "bytes": 8 * S * H * Dh})
        else:
            o, lse = attn_fwd(q, k, v, scale)
            do = rnd(1, S, H, Dh).bfloat16()
            run("attn_bwd", lambda: attn_bwd_native(q, k, v, o, lse, do, scale), {"flops": 2.5 * fl, "bytes": 16 * S * H * Dh})
    elif family == "conv":
        x = rnd(4, 176, 320, 256).bfloat16()
        w = (rnd(256, 256, 3, 3, 3) / (256 * 27) ** 0.5).bfloat16()
        pw, pb = F_.pack_conv_weight(w, torch.zeros(256, device=dev).bfloat16())
        run("conv3d", lambda: F_.conv3d_channels_last(x, pw, pb, (3, 3, 3)),
            {"flops": 2.0 * 4 * 176 * 320 * 256 * 256 * 27, "bytes": 2 * x.numel() * 2 + pw.numel() * 2})
    elif family == "masked_attention":
        # teacher forcing over [clean | noisy] halves: 2 x 10 frames of 880 tokens, 3-frame chunks, 6-chunk window
        from ..ops.attention_mask import masked_attention, teacher_forcing_segment_mask

        L, H, Dh = 10 * 880, 12, 128
        mask = teacher_forcing_segment_mask(L, 3 * 880, 6, 0, 0)
        q, k, v = (rnd(1, 2 * L, H, Dh).bfloat16() for _ in range(3))
        live = 4.0 * (2 * L) ** 2 * H * Dh * mask.density()
        with torch.no_grad():
            run("attn_fwd_masked", lambda: masked_attention(q, k, v, mask), {"flops": live, "bytes": 8 * 2 * L * H * Dh})
        qr = q.clone().requires_grad_(True)
        o = masked_attention(qr, k, v, mask)
        do = rnd(1, 2 * L, H, Dh).bfloat16()
        run("attn_bwd_masked", lambda: torch.autograd.grad(o, qr, do, retain_graph=True), {"flops": 2.5 * live, "bytes": 16 * 2 * L * H * Dh})
    elif family == "scatter":
        # the peer-scatter epilogues in their single-rank form (every "peer" is this GPU, nothing waits): what the
        # epilogue costs beside the plain kernel, without NVLink in the picture
        import ctypes

        from ..ops._lib import c_float, c_int, c_ll, load, ptr, stream_handle
        from ..ops.functional import status_word

        lib = load()
        M, D = 6820, 3072
        x, w = rnd(M, D).bfloat16(), (rnd(3 * D, D) / D ** 0.5).bfloat16()
        bias = torch.zeros(3 * D, device=dev, dtype=torch.bfloat16)
        qkv, recv = torch.empty(M, 3 * D, device=dev, dtype=torch.bfloat16), torch.empty(M, 3 * D, device=dev, dtype=torch.bfloat16)
        flag, counter = torch.zeros(4, device=dev, dtype=torch.int32), torch.zeros(1, device=dev, dtype=torch.int32)
        one = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())       # noqa: E731
        dst, flags = one(recv), one(flag)
        run("gemm_scatter(1 rank)", lambda: lib.solar_gemm_bf16_scatter(
            ptr(x), ptr(w), ptr(qkv), ptr(bias), c_int(M), c_int(3 * D), c_int(D), c_ll(D), c_ll(D), c_ll(3 * D), c_int(0),
            c_int(0), ptr(status_word(dev)), c_int(0), stream_handle(), dst, flags, ptr(counter), c_int(1), c_ll(3 * D),
            c_int(D), c_int(D), c_int(0), c_int(2 * D), c_int(0)),
            {"flops": 2.0 * M * 3 * D * D, "bytes": 2 * (M * D + 3 * D * D + M * 3 * D)})
        S, H, Dh = 16384, 6, 128
        q, k, v = (rnd(S, H * Dh).bfloat16() for _ in range(3))
        o, obuf = torch.empty(S, H * Dh, device=dev, dtype=torch.bfloat16), torch.empty(S, H * Dh, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(1, H, S, device=dev)
        starts = (ctypes.c_int * 2)(0, S)
        run("attn_fwd_scatter(1 rank)", lambda: lib.solar_attn_fwd_scatter(
            ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(S), c_int(S), c_int(H), c_int(Dh), c_ll(H * Dh), c_ll(H * Dh),
            c_ll(H * Dh), c_ll(H * Dh), c_float(1.0 / math.sqrt(Dh)), ptr(status_word(dev)), stream_handle(), one(obuf), flags,
            ptr(counter), c_int(1), c_ll(H * Dh), c_ll(S), starts, c_int(0)),
            {"flops": 4.0 * S * S * H * Dh, "bytes": 8 * S * H * Dh})
    elif family == "gemm":
        a, b = rnd(8192, 4096).bfloat16(), rnd(8192, 4096).bfloat16()
        run("gemm_nt", lambda: ops.gemm(a, b, ops.NT), {"flops": 2.0 * 8192 * 8192 * 4096, "bytes": 2 * (2 * 8192 * 4096 + 8192 * 8192)})
    else:
        raise SystemExit(f"unknown kernel family {family!r}")
    return plan


def wan5b_suite(seq=27280):
    d, f = 3072, 14336
    rows = []
    for (M, N, K, lay) in [(seq, 3 * d, d, "nt"), (seq, d, d, "nt"), (seq, f, d, "nt"), (seq, d, f, "nt"),
                           (seq, d, 3 * d, "nn"), (seq, d, f, "nn"), (seq, f, d, "nn"),
                           (3 * d, d, seq, "tn"), (f, d, seq, "tn"), (d, f, seq, "tn")]:
        rows.append(bench_gemm(M, N, K, lay, out_f32=(lay == "tn")))
    return rows


def tile_modes(seq=3410, iters=10):
    """Every GEMM of a Wan-5B block at ``seq`` rows per rank under each forced tile shape (CTA pair 256 x 256, one CTA
    128 x 256, one CTA 128 x 192) and under the launcher's own choice; each forced result is checked against the fp32
    product of the same operands."""
    from ..ops import _lib

    lib = _lib.load()
    d, f = 3072, 14336
    rows = []
    for (M, N, K, lay) in [(seq, 3 * d, d, "nt"), (seq, d, d, "nt"), (seq, f, d, "nt"), (seq, d, f, "nt"),
                           (seq, d, 3 * d, "nn"), (seq, d, f, "nn"), (seq, f, d, "nn"),
                           (3 * d, d, seq, "tn"), (f, d, seq, "tn"), (d, f, seq, "tn")]:
        layc = {"nt": ops.NT, "nn": ops.NN, "tn": ops.TN}[lay]
        g = torch.Generator(device="cuda").manual_seed(1)
        sa, sb = {"nt": ((M, K), (N, K)), "nn": ((M, K), (K, N)), "tn": ((K, M), (K, N))}[lay]
        a = torch.randn(sa, device="cuda", generator=g).bfloat16()
        b = torch.randn(sb, device="cuda", generator=g).bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.float32 if lay == "tn" else torch.bfloat16)
        af, bf = a[:256].float() if lay != "tn" else a[:, :256].float(), b.float()
        want = {"nt": lambda: af @ bf.t(), "nn": lambda: af @ bf, "tn": lambda: af.t() @ bf}[lay]()
        row = {"layout": lay, "M": M, "N": N, "K": K}
        for name, mode in (("pair256", 1), ("pair128", 3), ("single256", 0), ("single192", 2), ("auto", -1)):
            old = lib.solar_gemm_pair_mode(mode)
            try:
                ms = time_fn(lambda: ops.gemm(a, b, layc, out=out), iters)
                err = float((out[:256].float() - want).abs().max() / want.abs().max())
            finally:
                lib.solar_gemm_pair_mode(old)
            row[name + "_ms"] = round(ms, 4)
            row[name + "_rel_err"] = round(err, 5)
        row["tflops_auto"] = round(2.0 * M * N * K / row["auto_ms"] / 1e9, 1)
        rows.append(row)
    ops.check_status()
    return rows


def bwd_trace(seq=8192, heads=12, head_dim=128):
    """Cycle counters the attention-backward kernels keep for CTA (0, 0, 0) of each launch (``clock64`` deltas of
    its roles), read back after one backward pass."""
    import ctypes

    from ..ops import _lib
    from ..ops.attention_native import attn_bwd, attn_fwd

    lib = _lib.load()
    lib.solar_attn_bwd_trace.argtypes = [ctypes.c_int, ctypes.c_void_p]
    q, k, v = (torch.randn(1, seq, heads, head_dim, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    o, lse = attn_fwd(q, k, v, head_dim ** -0.5)
    do = torch.randn_like(o)
    lib.solar_attn_bwd_trace(1, None)
    attn_bwd(q, k, v, o, lse, do, head_dim ** -0.5)
    torch.cuda.synchronize()
    out = (ctypes.c_longlong * 32)()
    lib.solar_attn_bwd_trace(0, out)
    return {"seq": seq, "heads": heads, "head_dim": head_dim, "counters": list(out)}


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=4096)
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--layout", default="nt")
    g.add_argument("--f32", action="store_true")
    g.add_argument("--iters", type=int, default=10)
    a = sub.add_parser("attention")
    a.add_argument("--seq", type=int, default=8192)
    a.add_argument("--kv", type=int, default=None)
    a.add_argument("--heads", type=int, default=24)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--backward", action="store_true")
    a.add_argument("--iters", type=int, default=5)
    r = sub.add_parser("rowops")
    r.add_argument("--rows", type=int, default=27280)
    r.add_argument("--dim", type=int, default=3072)
    c = sub.add_parser("conv")
    c.add_argument("--frames", type=int, default=4)
    c.add_argument("--height", type=int, default=176)
    c.add_argument("--width", type=int, default=320)
    c.add_argument("--cin", type=int, default=256)
    c.add_argument("--cout", type=int, default=256)
    c.add_argument("--iters", type=int, default=5)
    s = sub.add_parser("suite")
    s.add_argument("--seq", type=int, default=27280)
    bt = sub.add_parser("bwd-trace")
    bt.add_argument("--seq", type=int, default=8192)
    bt.add_argument("--heads", type=int, default=12)
    tl = sub.add_parser("tiles")
    tl.add_argument("--seq", type=int, default=3410)
    tl.add_argument("--iters", type=int, default=10)
    pr = sub.add_parser("probe")
    pr.add_argument("--family", required=True)
    pr.add_argument("--rows", type=int, default=27280)
    pr.add_argument("--dim", type=int, default=3072)
    args = ap.parse_args()
    if args.cmd == "probe":
        print(json.dumps({"family": args.family, "per_launch": probe(args.family, args.rows, args.dim)}))
        ops.check_status()
        return
    if args.cmd == "bwd-trace":
        print(json.dumps(bwd_trace(args.seq, args.heads)))
        return
    if args.cmd == "tiles":
        for row in tile_modes(args.seq, args.iters):
            print(json.dumps(row))
        return
    if args.cmd == "gemm":
        print(json.dumps(bench_gemm(args.m, args.n, args.k, args.layout, args.f32, args.iters)))
    elif args.cmd == "attention":
        print(json.dumps(bench_attention(args.seq, args.heads, args.head_dim, args.kv, args.backward, args.iters)))
    elif args.cmd == "conv":
        print(json.dumps(bench_conv(args.frames, args.height, args.width, args.cin, args.cout, iters=args.iters)))
    elif args.cmd == "rowops":
        for row in bench_rowops(args.rows, args.dim):
            print(json.dumps(row))
    else:
        for row in wan5b_suite(args.seq):
            print(json.dumps(row))
        for row in bench_rowops(args.seq, 3072):
            print(json.dumps(row))
    ops.check_status()


if __name__ == "__main__":
    main()
