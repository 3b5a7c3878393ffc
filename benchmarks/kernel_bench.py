"""Time the memory-bound kernels on benchmark-sized inputs and report achieved bandwidth against the roofline.

    python -m benchmarks.kernel_bench [--only NAME[,NAME...]] [--iters 20] [--small] [--out FILE]

Each case launches one kernel entry point on inputs larger than the L2 (so DRAM figures mean something), is
timed with CUDA events after warm-up (median), and reports ``GB/s = algorithmic bytes / time`` and the fraction of
the measured HBM copy bandwidth (``MEASURED_PEAKS.json`` at the repository root; 6450 GB/s otherwise).
``--small`` shrinks every case to a few hundred MB for profiler captures.  One JSON line per case.
"""
from __future__ import annotations

import argparse
import json

import torch


def _cases(small: bool):
    from ferrum_b200 import _lib, optim
    from ferrum_b200.ops import functional as F

    R = 4096 if small else 8192
    C = 4096
    dev = "cuda"
    bf = torch.bfloat16
    x32 = torch.randn(R, C, device=dev)
    xb = x32.to(bf)
    gb = torch.randn(R, C, device=dev).to(bf)
    gamma = torch.rand(C, device=dev) + 0.5
    beta = torch.randn(C, device=dev)
    cases = {}

    def case(name, fn, nbytes, note=""):
        cases[name] = (fn, nbytes, note)

    n = R * C
    case("unary_gelu_fwd_bf16", lambda: F.raw_unary(xb, "gelu"), n * 4, "K2")
    case("unary_gelu_bwd_bf16", lambda: F.raw_unary_bwd(gb, xb, "gelu"), n * 6, "K2 bwd")
    case("unary_relu_fwd_f32", lambda: F.raw_unary(x32, "relu"), n * 8, "K2")
    case("scalar_affine_f32", lambda: F.raw_unary(x32, "affine", 2.0, 1.0), n * 8, "K3 / Normalize")
    y32 = torch.randn(R, C, device=dev)
    case("binary_add_f32", lambda: F.raw_binary(x32, y32, "add"), n * 12, "K1")
    case("binary_bcast_row_f32", lambda: F.raw_binary(x32, beta, "add"), n * 8, "K1 [B,F]+[F]")
    case("cast_f32_to_bf16", lambda: F.raw_cast(x32, bf), n * 6, "cast")
    case("transpose_bf16", lambda: F.transpose_2d(xb), n * 4, "K5t")
    case("reduce_sum_all_f32", lambda: F.raw_reduce(x32, "sum", None), n * 4, "K4 full")
    case("reduce_sum_rows_f32", lambda: F.raw_reduce(x32, "sum", 1), n * 4, "K4 row")
    case("reduce_sum_cols_f32", lambda: F.raw_reduce(x32, "sum", 0), n * 4, "K4 column")
    case("argmax_rows_f32", lambda: F.arg_reduce(x32, True, 1), n * 4, "K4 arg")
    case("colsum_bf16", lambda: F.raw_colsum(xb), n * 2, "bias gradient")

    lib = _lib.cuda()
    st = lambda: torch.cuda.current_stream().cuda_stream  # noqa: E731
    yb = torch.empty_like(xb)
    mean = torch.empty(R, device=dev)
    rstd = torch.empty(R, device=dev)

    def ln_fwd():
        lib.fb_layernorm_fwd(xb.data_ptr(), gamma.data_ptr(), beta.data_ptr(), yb.data_ptr(), mean.data_ptr(),
                             rstd.data_ptr(), R, C, 1e-5, 2, 3, st())

    ln_fwd()
    nblk = lib.fb_layernorm_bwd_blocks(R, C)
    partial = torch.empty(max(nblk, 1), 3, C, device=dev)
    stats = torch.zeros(3, C, device=dev)
    dxb = torch.empty_like(xb)

    def ln_bwd():
        lib.fb_layernorm_bwd(gb.data_ptr(), xb.data_ptr(), None, gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                             dxb.data_ptr(), partial.data_ptr(), stats.data_ptr(), R, C, 2, 3, nblk, 1, st())

    def ln_fwd_plain():
        lib.fb_layernorm_fwd(xb.data_ptr(), gamma.data_ptr(), beta.data_ptr(), yb.data_ptr(), mean.data_ptr(),
                             rstd.data_ptr(), R, C, 1e-5, 0, 3, st())

    dact = torch.rand(R, C, device=dev).to(bf)

    def ln_bwd_stored():
        lib.fb_layernorm_bwd(gb.data_ptr(), xb.data_ptr(), dact.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                             rstd.data_ptr(), dxb.data_ptr(), partial.data_ptr(), stats.data_ptr(), R, C, 0, 3, nblk, 1,
                             st())

    case("layernorm_gelu_fwd_bf16", ln_fwd, n * 4, "K7 fused GELU+LN")
    case("layernorm_gelu_bwd_bf16", ln_bwd, n * 6, "K7 bwd + dgamma/dbeta/colsum")
    case("layernorm_fwd_bf16", ln_fwd_plain, n * 4, "K7 (activation done by the GEMM epilogue)")
    case("layernorm_bwd_stored_act_bf16", ln_bwd_stored, n * 8, "K7 bwd, act'(z) read from memory")

    Cs = 1000
    lg = torch.randn(R, Cs, device=dev).to(bf)
    labels = torch.randint(0, Cs, (R,), device=dev)
    rl = torch.empty(R, device=dev)
    dl = torch.empty_like(lg)
    case("softmax_fwd_bf16_1000", lambda: F.softmax(lg, -1), R * Cs * 4, "K6")
    case("cross_entropy_fused_bf16_1000",
         lambda: lib.fb_ce_fwd_bwd(lg.data_ptr(), labels.data_ptr(), rl.data_ptr(), dl.data_ptr(), R, Cs, 1.0 / R, 3, 3,
                                   st()), R * Cs * 4, "K6b loss + dlogits")
    p32 = torch.rand(R, C, device=dev) * 0.9 + 0.05
    t32 = torch.rand(R, C, device=dev)
    case("mse_loss_fwd_f32", lambda: F.elementwise_loss(p32, t32, "mse"), n * 8, "K11")
    bx = torch.randn(R, 1024, device=dev)
    bg_, bb_ = torch.ones(1024, device=dev), torch.zeros(1024, device=dev)
    rm, rv = torch.zeros(1024, device=dev), torch.ones(1024, device=dev)
    case("batchnorm_fwd_f32", lambda: F.batch_norm(bx, bg_, bb_, rm, rv, True), R * 1024 * 4 * 3, "K8 (one statistics pass + apply: 2 reads + 1 write)")
    case("dropout_fwd_bf16", lambda: F.dropout(xb, 0.1, True, seed=1), n * 5, "K9 (+1 B mask)")

    V, D, S, Bt = 50000, 1024, 256, 128 if small else 512
    w = torch.randn(V, D, device=dev)
    from ferrum_b200.data import zipf_indices

    idx = torch.from_numpy(zipf_indices(V, 1.1, Bt * S, seed=0)).to(dev).reshape(Bt, S)
    case("embedding_meanpool_fwd", lambda: F.embedding_mean_pool(w, idx, bf), Bt * S * D * 4, "K10 gather+pool")
    gout = torch.randn(Bt, D, device=dev).to(bf)
    sidx, perm = torch.sort(idx.reshape(-1), stable=True)
    dw = torch.zeros(V, D, device=dev)
    case("embedding_scatter_add_bwd",
         lambda: lib.fb_embedding_bwd_sorted(gout.data_ptr(), sidx.data_ptr(), perm.data_ptr(), dw.data_ptr(),
                                             Bt * S, D, S, 1.0 / S, -1, V, 3, st()), Bt * S * D * 2, "K10 bwd")
    gi = torch.randint(0, R, (R,), device=dev)
    case("gather_rows_f32", lambda: F.gather_rows(x32, gi), n * 8, "K18 collate")

    P = (32 << 20) if small else (125 << 20)
    pp = torch.randn(P, device=dev, requires_grad=True)
    pp.grad = torch.randn(P, device=dev) * 1e-2
    adam = optim.Adam([pp], optim.AdamConfig(lr=3e-4))
    adam.step()
    case("adam_multi_tensor", adam.step, P * 28, "K12 (g,p,m,v read; p,m,v write)")
    sgd = optim.SGD([pp], optim.SGDConfig(lr=0.1, momentum=0.9))
    sgd.step()
    case("sgd_momentum_multi_tensor", sgd.step, P * 20, "K12")
    gsc = optim.GradScaler.with_scale(2.0)
    case("amp_unscale_check", lambda: gsc.unscale_gradients([pp]), P * 8, "K17")
    case("amp_clip_grad_norm", lambda: optim.clip_grad_norm([pp], 1e9), P * 4, "K17 (sum of squares pass)")

    # secondary layers: recurrent gate kernels, convolution window matrix, pooling, attention
    Bq, Hq = (2048 if small else 8192), 1024
    xi4, hh4 = torch.randn(Bq, 4 * Hq, device=dev), torch.randn(Bq, 4 * Hq, device=dev)
    cprev = torch.randn(Bq, Hq, device=dev)
    case("lstm_gates_fwd_f32", lambda: F.lstm_gates(xi4, hh4, cprev), Bq * Hq * 4 * (8 + 1 + 2 + 4),
         "K15 (2 x [B,4H] + c read; h, c, 4 gate activations written)")
    xi3, hh3 = torch.randn(Bq, 3 * Hq, device=dev), torch.randn(Bq, 3 * Hq, device=dev)
    case("gru_gates_fwd_f32", lambda: F.gru_gates(xi3, hh3, cprev), Bq * Hq * 4 * (6 + 1 + 1 + 3),
         "K15 (2 x [B,3H] + h read; h' and r, z, n written)")
    img = torch.randn(16 if small else 64, 64, 56, 56, device=dev)
    case("im2col_3x3_f32", lambda: F.im2col(img, (3, 3), (1, 1), (1, 1), (1, 1)),
         img.numel() * 4 * (1 + 9), "K14 (input read once, 9x window matrix written)")
    # 3 x 3 convolution, 64 -> 64 channels, padding 1, bf16 autocast: window matrix + GEMM against the implicit GEMM
    import ferrum_b200 as fb_
    wconv = (torch.randn(64, 64, 3, 3, device=dev) * 0.05).requires_grad_(True)
    bconv = torch.zeros(64, device=dev, requires_grad=True)
    imgg = img.detach().clone().requires_grad_(True)
    gconv = torch.randn_like(img)
    conv_bytes = img.numel() * 4 * 2   # NCHW fp32 input read, NCHW fp32 output written (64 -> 64 channels)

    def conv_window(train):
        with fb_.autocast():
            cols = F.im2col(imgg if train else img, (3, 3), (1, 1), (1, 1), (1, 1))
            y = F.linear(cols, wconv.reshape(64, -1), bconv).reshape(img.shape[0], 56 * 56, 64)
            y = y.transpose(1, 2).reshape(img.shape[0], 64, 56, 56)
        return torch.autograd.grad(y, (imgg, wconv, bconv), gconv) if train else y

    def conv_implicit(train):
        with fb_.autocast():
            y = F.conv2d_igemm(imgg if train else img, wconv, bconv, (1, 1), (1, 1))
        return torch.autograd.grad(y, (imgg, wconv, bconv), gconv) if train else y

    # the same input through a stride-2 3 x 3 convolution, 64 -> 128 channels (a down-sampling layer)
    wdown = (torch.randn(128, 64, 3, 3, device=dev) * 0.05).requires_grad_(True)
    bdown = torch.zeros(128, device=dev, requires_grad=True)
    gdown = torch.randn(img.shape[0], 128, 28, 28, device=dev)
    down_bytes = img.numel() * 4 + gdown.numel() * 4

    def down_window(train):
        with fb_.autocast():
            cols = F.im2col(imgg if train else img, (3, 3), (2, 2), (1, 1), (1, 1))
            y = F.linear(cols, wdown.reshape(128, -1), bdown).reshape(img.shape[0], 28 * 28, 128)
            y = y.transpose(1, 2).reshape(img.shape[0], 128, 28, 28)
        return torch.autograd.grad(y, (imgg, wdown, bdown), gdown) if train else y

    def down_implicit(train):
        with fb_.autocast():
            y = F.conv2d_igemm(imgg if train else img, wdown, bdown, (1, 1), (1, 1), (2, 2))
        return torch.autograd.grad(y, (imgg, wdown, bdown), gdown) if train else y

    case("conv2d_3x3_s2_fwd_bwd_window_matrix_bf16", lambda: down_window(True), 3 * down_bytes,
         "K14 stride 2, 64 -> 128 channels: im2col + GEMMs + col2im")
    case("conv2d_3x3_s2_fwd_bwd_implicit_gemm_bf16", lambda: down_implicit(True), 3 * down_bytes,
         "K14 stride 2, 64 -> 128 channels: space-to-depth layout + implicit GEMMs in all three directions")
    case("conv2d_3x3_fwd_window_matrix_bf16", lambda: conv_window(False), conv_bytes,
         "K14 im2col (9x matrix) + tcgen05 GEMM + transpose back")
    case("conv2d_3x3_fwd_implicit_gemm_bf16", lambda: conv_implicit(False), conv_bytes,
         "K14 NHWC bf16 copy + implicit GEMM (4-D TMA boxes per filter tap) + NCHW copy")
    case("conv2d_3x3_fwd_bwd_window_matrix_bf16", lambda: conv_window(True), 3 * conv_bytes,
         "K14 forward + backward through the stored window matrix (col2im for the data gradient)")
    case("conv2d_3x3_fwd_bwd_implicit_gemm_bf16", lambda: conv_implicit(True), 3 * conv_bytes,
         "K14 forward + data gradient + weight gradient as implicit GEMMs")
    case("maxpool2d_2x2_f32", lambda: F.pool2d(img, (2, 2), (2, 2), "max"), img.numel() * 4 * 1.25 + img.numel(),
         "K14 (input read, quarter-size output + int32 argmax written)")
    Ba, Ha, Sa, Da = (2 if small else 8), 16, 1024, 64
    qa = torch.randn(Ba, Sa, Ha, Da, device=dev).to(bf).permute(0, 2, 1, 3)
    ka = torch.randn(Ba, Sa, Ha, Da, device=dev).to(bf).permute(0, 2, 1, 3)
    va = torch.randn(Ba, Sa, Ha, Da, device=dev).to(bf).permute(0, 2, 1, 3)

    def attn():
        import ferrum_b200 as fb
        with fb.autocast():
            p_ = F.softmax(F.bmm_scaled(qa, ka.transpose(-1, -2), Da ** -0.5), -1)
            return F.bmm_scaled(p_, va, 1.0, heads_inner=True)

    case("attention_fwd_bf16_S1024_D64", attn, Ba * Ha * Sa * Sa * 2 * 4 + 4 * Ba * Ha * Sa * Da * 2,
         "K16 (batched tcgen05 QK^T, row softmax, batched PV; bytes = score matrix written + read twice + q, k, v, o)")
    case("attention_flash_fwd_bf16_S1024_D64", lambda: F.flash_attention(qa, ka, va, Da ** -0.5),
         4 * Ba * Ha * Sa * Da * 2, "K16 blockwise tcgen05 attention (bytes = q, k, v, o only)")
    q128, k128, v128 = (torch.randn(Ba, Sa, Ha // 2, 128, device=dev).to(bf).permute(0, 2, 1, 3) for _ in range(3))

    def attn128():
        import ferrum_b200 as fb
        with fb.autocast():
            p_ = F.softmax(F.bmm_scaled(q128, k128.transpose(-1, -2), 128 ** -0.5), -1)
            return F.bmm_scaled(p_, v128, 1.0, heads_inner=True)

    case("attention_fwd_bf16_S1024_D128", attn128, Ba * (Ha // 2) * Sa * Sa * 2 * 4 + 4 * Ba * (Ha // 2) * Sa * 128 * 2,
         "K16 head dimension 128, 8 heads (batched tcgen05 QK^T, row softmax, batched PV)")
    case("attention_flash_fwd_bf16_S1024_D128", lambda: F.flash_attention(q128, k128, v128, 128 ** -0.5),
         4 * Ba * (Ha // 2) * Sa * 128 * 2, "K16 blockwise tcgen05 attention, head dimension 128 (bytes = q, k, v, o only)")
    # training direction: forward + backward of the attention core, gradients with respect to q, k, v
    go = torch.randn(Ba, Sa, Ha, Da, device=dev).to(bf).permute(0, 2, 1, 3)  # laid out like the outputs
    import ferrum_b200 as fb

    qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (qa, ka, va))

    def attn_train_materialised():
        with fb.autocast():
            p_ = F.softmax(F.bmm_scaled(qg, kg.transpose(-1, -2), Da ** -0.5), -1)
            out = F.bmm_scaled(p_, vg, 1.0, heads_inner=True)
            return torch.autograd.grad(out, (qg, kg, vg), go)

    def attn_train_blockwise():
        return torch.autograd.grad(F.attention_blockwise(qg, kg, vg, Da ** -0.5), (qg, kg, vg), go)

    q128g, k128g, v128g = (t.detach().clone().requires_grad_(True) for t in (q128, k128, v128))
    go128 = torch.randn(Ba, Sa, Ha // 2, 128, device=dev).to(bf).permute(0, 2, 1, 3)

    def attn128_train_materialised():
        with fb.autocast():
            p_ = F.softmax(F.bmm_scaled(q128g, k128g.transpose(-1, -2), 128 ** -0.5), -1)
            out = F.bmm_scaled(p_, v128g, 1.0, heads_inner=True)
            return torch.autograd.grad(out, (q128g, k128g, v128g), go128)

    case("attention_fwd_bwd_materialised_bf16_S1024_D128", attn128_train_materialised,
         Ba * (Ha // 2) * Sa * Sa * 2 * 10 + 12 * Ba * (Ha // 2) * Sa * 128 * 2,
         "K16 head dimension 128: forward + backward through the stored S x S probabilities")
    case("attention_fwd_bwd_blockwise_bf16_S1024_D128",
         lambda: torch.autograd.grad(F.attention_blockwise(q128g, k128g, v128g, 128 ** -0.5), (q128g, k128g, v128g),
                                     go128),
         12 * Ba * (Ha // 2) * Sa * 128 * 2, "K16 head dimension 128: blockwise tcgen05 forward + backward")
    case("attention_fwd_bwd_materialised_bf16_S1024_D64", attn_train_materialised,
         Ba * Ha * Sa * Sa * 2 * 10 + 12 * Ba * Ha * Sa * Da * 2,
         "K16 forward + backward through the stored S x S probabilities (batched GEMMs, softmax and its backward)")
    case("attention_fwd_bwd_blockwise_bf16_S1024_D64", attn_train_blockwise, 12 * Ba * Ha * Sa * Da * 2,
         "K16 blockwise tcgen05 forward + backward (bytes = q, k, v, o, dO, dq, dk, dv and the re-read operands)")
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    from ferrum_b200.utils.profiler import measured_peaks
    from ferrum_b200.utils.runtime import check_status

    pk = measured_peaks()
    hbm = pk["hbm_gbs"] if pk else 6450.0
    cases = _cases(a.small)
    only = [s for s in a.only.split(",") if s]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    results = []
    for name, (fn, nbytes, note) in cases.items():
        if only and name not in only:
            continue
        try:
            for _ in range(a.warmup):
                fn()
        except Exception as exc:  # noqa: BLE001 - report and go on with the other kernels
            print(json.dumps({"kernel": name, "error": f"{type(exc).__name__}: {exc}"}), flush=True)
            continue
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        ms = ts[len(ts) // 2]
        res = {"kernel": name, "row": note, "us": 1e3 * ms, "algorithmic_MB": nbytes / 1e6,
               "GBps": nbytes / ms / 1e6, "frac_of_measured_hbm" if pk else "frac_of_fallback_hbm":
               nbytes / ms / 1e6 / hbm}
        results.append(res)
        print(json.dumps(res), flush=True)
    check_status()
    if a.out:
        with open(a.out, "w") as f:
            json.dump(results, f, indent=1)


if __name__ == "__main__":
    main()
