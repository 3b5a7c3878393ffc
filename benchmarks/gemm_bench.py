"""Time the tcgen05 GEMM on one shape (also the small case used for kernel profiles).

    python -m benchmarks.gemm_bench --m 8192 --n 4096 --k 4096 --layout nt --iters 20 [--cublas]

``--layout``: ``nt`` forward (A, B K-major), ``nn`` dgrad (B MN-major), ``tn`` wgrad (both MN-major, fp32 out).
Prints one JSON line: median CUDA-event time after warm-up with an L2 flush between iterations, TFLOP/s, and the
fraction of the measured cuBLAS bf16 peak when ``MEASURED_PEAKS.json`` is present at the repository root.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--act", default=None)
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--simt", action="store_true",
                    help="the exact-fp32 SIMT kernel (FFMA pipe; compared with cuBLAS fp32 without TF32)")
    ap.add_argument("--tf32", action="store_true", help="fp32 operands on the tensor cores (kind::tf32, fp32 output)")
    ap.add_argument("--prof", action="store_true",
                    help="CTA-pair kernel: report where the MMA thread waits (drained accumulator / operands) and how long "
                         "an epilogue warp is busy, averaged over the pairs of the last launch")
    ap.add_argument("--dual", action="store_true", help="also store act'(z) (second bf16 output; needs --act)")
    ap.add_argument("--two-cta", action="store_true", help="use the CTA-pair (cta_group::2) kernel")
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul (cuBLAS) on the same operands")
    ap.add_argument("--out", default=None, choices=["bf16", "fp32"],
                    help="result dtype of the bf16 GEMM (default: fp32 for the tn layout, bf16 otherwise)")
    ap.add_argument("--accumulate", action="store_true", help="add the product to the existing fp32 result")
    ap.add_argument("--group-m", type=int, default=0,
                    help="CTA-pair kernel: 256-row blocks per rasterisation group (default: the library's)")
    a = ap.parse_args()

    from ferrum_b200.ops import gemm as _g
    from ferrum_b200.ops.gemm import gemm_bf16, gemm_f32, gemm_tf32

    _g.set_gemm_2cta(a.two_cta)
    from ferrum_b200.utils.runtime import check_status

    M, N, K = a.m, a.n, a.k
    a_mn = a.layout == "tn"
    b_mn = a.layout in ("nn", "tn")
    A = torch.randn(K, M, device="cuda").to(torch.bfloat16).t() if a_mn else torch.randn(M, K, device="cuda").to(
        torch.bfloat16)
    B = torch.randn(K, N, device="cuda").to(torch.bfloat16).t() if b_mn else torch.randn(N, K, device="cuda").to(
        torch.bfloat16)
    f32_out = (a.out == "fp32") if a.out is not None else a.layout == "tn"
    out = torch.zeros(M, N, device="cuda", dtype=torch.float32 if (f32_out or a.tf32 or a.simt) else torch.bfloat16)
    if a.group_m > 0:
        from ferrum_b200 import _lib as _l0

        _l0.cuda().fb_gemm_bf16_2cta_set_group_m(a.group_m)
    if a.tf32 or a.simt:
        A, B = A.float().t().contiguous().t() if a_mn else A.float(), B.float().t().contiguous().t() if b_mn else B.float()
    bias = torch.randn(N, device="cuda") if a.bias else None
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn):
        for _ in range(a.warmup):
            fn()
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
        return ts[len(ts) // 2]

    aux = torch.empty_like(out) if a.dual else None
    if a.simt:
        ms = timeit(lambda: gemm_f32(A, B, bias=bias, act=a.act, out=out))
    elif a.tf32:
        ms = timeit(lambda: gemm_tf32(A, B, bias=bias, act=a.act, out=out, kernel="2cta" if a.two_cta else "1cta"))
    else:
        ms = timeit(lambda: gemm_bf16(A, B, bias=bias, act=a.act, out=out, act_grad=aux, accumulate=a.accumulate))
    check_status()
    flops = 2.0 * M * N * K
    if a.two_cta and not a.accumulate:
        ref = (A[:256].float() @ B.float().t())
        if bias is not None:
            ref = ref + bias
        if a.act == "gelu":
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        elif a.act == "relu":
            ref = torch.relu(ref)
        res_err = (out[:256].float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
    res = {"kernel": "gemm_f32_simt" if a.simt else ("gemm_tf32_tcgen05_2cta" if a.two_cta else "gemm_tf32_tcgen05") if a.tf32 else "gemm_bf16_tcgen05_2cta" if a.two_cta else "gemm_bf16_tcgen05", "M": M, "N": N, "K": K, "layout": a.layout, "out": str(out.dtype).replace("torch.", ""), "ms": ms,
           "tflops": flops / ms / 1e9}
    if a.two_cta and not a.accumulate:
        res["rel_err_first_rows"] = res_err
    if a.simt:
        ref = (A[:256].double() @ B.double().t()).float()
        res["rel_err_first_rows"] = (out[:256] - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        # FFMA ceiling of this GPU: SMs x 128 lanes x 2 flops x clock (the clock is whatever the run gets)
        res["ffma_peak_tflops_at_max_clock"] = 148 * 128 * 2 * 1.965e9 / 1e12
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        pk = json.load(open(peaks))
        res["frac_of_measured_bf16_burst"] = res["tflops"] / pk["bf16_tflops"]
    if a.cublas:
        torch.backends.cuda.matmul.allow_tf32 = False
        if a.tf32:
            torch.backends.cuda.matmul.allow_tf32 = True  # compare against cuBLAS' TF32 path, not its fp32 SIMT one
        Ac, Bc = A.contiguous(), B.contiguous()
        cms = timeit(lambda: torch.matmul(Ac, Bc.t()))
        res["cublas_ms"], res["cublas_tflops"] = cms, flops / cms / 1e9
    if a.prof and a.two_cta:
        from ferrum_b200 import _lib

        lib = _lib.cuda()
        pairs = lib.fb_gemm_bf16_2cta_pairs()
        buf = torch.zeros(pairs * 4, dtype=torch.int64, device="cuda")
        lib.fb_gemm_bf16_2cta_set_profile(buf.data_ptr())
        gemm_bf16(A, B, bias=bias, act=a.act, out=out, act_grad=aux)
        torch.cuda.synchronize()
        lib.fb_gemm_bf16_2cta_set_profile(None)
        t = buf.view(pairs, 4).double().mean(0) / 1e3
        res["prof_us"] = {"mma_waits_accumulator": t[0].item(), "mma_waits_operands": t[1].item(),
                          "epilogue_warp_busy": t[2].item(), "kernel": t[3].item()}
    print(json.dumps(res))


if __name__ == "__main__":
    main()
