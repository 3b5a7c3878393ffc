"""tcgen05 GEMM and SIMT GEMM against a plain fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, bias, act):
    y = a.float() @ b.float().t()
    if bias is not None:
        y = y + bias
    if act == "relu":
        y = torch.relu(y)
    elif act == "gelu":
        y = torch.nn.functional.gelu(y, approximate="tanh")
    elif act == "silu":
        y = torch.nn.functional.silu(y)
    return y


def _mk(rows, cols, mn_major, scale=1.0):
    """bf16 [rows(MN), cols(K)] view, stored K-major or MN-major."""
    if mn_major:
        return (torch.randn(cols, rows, device="cuda") * scale).to(torch.bfloat16).t()
    return (torch.randn(rows, cols, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (384, 200, 328), (136, 72, 1000),
                                   (1024, 1000, 4096)])
def test_gemm_bf16_layouts(a_mn, b_mn, M, N, K):
    from ferrum_b200.ops.gemm import gemm_bf16
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(M * 7 + N * 3 + K + a_mn * 2 + b_mn)
    a = _mk(M, K, a_mn, 0.5)
    b = _mk(N, K, b_mn, 0.5)
    out = gemm_bf16(a, b, out_dtype=torch.float32)
    check_status()
    ref = _ref(a, b, None, None)
    err = (out - ref).abs().max().item()
    tol = 2e-3 * (K ** 0.5) * 0.25 + 1e-3
    assert err < tol, f"max err {err} (tol {tol}) for {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}"


@pytest.mark.parametrize("act", [None, "relu", "gelu", "silu"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_bf16_epilogue(act, out_dtype):
    from ferrum_b200.ops.gemm import gemm_bf16
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(1)
    M, N, K = 300, 520, 192
    a = _mk(M, K, 0, 0.3)
    b = _mk(N, K, 0, 0.3)
    bias = torch.randn(N, device="cuda")
    out = gemm_bf16(a, b, bias=bias, act=act, out_dtype=out_dtype)
    check_status()
    ref = _ref(a, b, bias, act)
    tol = 3e-2 if out_dtype == torch.bfloat16 else 5e-3
    assert (out.float() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())


def test_gemm_bf16_accumulate():
    from ferrum_b200.ops.gemm import gemm_bf16
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(2)
    a = _mk(256, 128, 1, 0.3)
    b = _mk(264, 128, 1, 0.3)
    out = torch.randn(256, 264, device="cuda")
    ref = out + _ref(a, b, None, None)
    gemm_bf16(a, b, out=out, accumulate=True)
    check_status()
    assert (out - ref).abs().max().item() < 5e-3


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_f32_simt(ta, tb):
    from ferrum_b200.ops.gemm import gemm_f32

    torch.manual_seed(3)
    M, N, K = 70, 45, 33
    a = torch.randn(K, M, device="cuda").t() if ta else torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda").t() if tb else torch.randn(N, K, device="cuda")
    bias = torch.randn(N, device="cuda")
    out = gemm_f32(a, b, bias=bias, act="relu")
    ref = torch.relu(a @ b.t() + bias)
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 16), (64, 64, 20), (300, 520, 100), (257, 132, 64), (1000, 1024, 516)])
def test_gemm_f32_simt_fast_path(ta, tb, M, N, K):
    """The register-tiled fp32 kernel (regular operands: unit stride along K or along M / N, 16-byte aligned
    pitch) against a float64 product, with bias, activation and accumulation, ragged edges in every dimension."""
    from ferrum_b200.ops.gemm import gemm_f32

    torch.manual_seed(M + N + K)
    a = torch.randn(K, M, device="cuda").t() if ta else torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda").t() if tb else torch.randn(N, K, device="cuda")
    bias = torch.randn(N, device="cuda")
    ref = (a.double() @ b.double().t())
    out = gemm_f32(a, b)
    assert (out - ref.float()).abs().max().item() < 2e-4 * K ** 0.5
    out = gemm_f32(a, b, bias=bias, act="relu")
    assert (out - torch.relu(ref + bias).float()).abs().max().item() < 2e-4 * K ** 0.5
    acc = torch.ones(M, N, device="cuda")
    gemm_f32(a, b, out=acc, accumulate=True)
    assert (acc - (1 + ref).float()).abs().max().item() < 2e-4 * K ** 0.5


def test_gemm_f32_simt_fast_path_batched_and_strided_output():
    from ferrum_b200.ops.gemm import gemm_f32

    torch.manual_seed(8)
    a = torch.randn(3, 130, 64, device="cuda")
    b = torch.randn(3, 96, 64, device="cuda")
    out = gemm_f32(a, b)
    assert torch.allclose(out, a @ b.transpose(1, 2), atol=2e-4, rtol=1e-4)
    wide = torch.zeros(130, 200, device="cuda")
    gemm_f32(a[0], b[0], out=wide[:, 8:104])  # row pitch 200, column offset 8: 16-byte aligned, not contiguous
    assert torch.allclose(wide[:, 8:104], a[0] @ b[0].t(), atol=2e-4, rtol=1e-4)
    assert wide[:, :8].abs().sum().item() == 0 and wide[:, 104:].abs().sum().item() == 0


def test_gemm_f32_batched():
    from ferrum_b200.ops.gemm import gemm_f32

    torch.manual_seed(4)
    a = torch.randn(3, 17, 29, device="cuda")
    b = torch.randn(3, 11, 29, device="cuda")
    out = gemm_f32(a, b)
    assert torch.allclose(out, a @ b.transpose(1, 2), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (512, 512, 256), (1024, 1000, 520), (776, 264, 1000),
                                   (2048, 4096, 1024), (4096, 4096, 256), (8192, 4096, 128)])
def test_gemm_bf16_cta_pair_kernel(a_mn, b_mn, M, N, K):
    """cta_group::2 kernel (256x256 and 256x128 tiles per CTA pair, chosen by wave fill) against the fp32
    reference, all operand layouts."""
    from ferrum_b200.ops import gemm as g
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(M + N + K + a_mn * 2 + b_mn)
    a = _mk(M, K, a_mn, 0.5)
    b = _mk(N, K, b_mn, 0.5)
    bias = torch.randn(N, device="cuda")
    prev = g._use_2cta
    g.set_gemm_2cta(True)
    try:
        out = g.gemm_bf16(a, b, bias=bias, out_dtype=torch.float32)
        acc = torch.ones(M, N, device="cuda")
        g.gemm_bf16(a, b, out=acc, accumulate=True)
        outb = g.gemm_bf16(a, b, act="relu")
        check_status()
    finally:
        g.set_gemm_2cta(prev)
    ref = _ref(a, b, bias, None)
    tol = 2e-3 * (K ** 0.5) * 0.25 + 1e-3
    assert (out - ref).abs().max().item() < tol
    assert (acc - (1.0 + _ref(a, b, None, None))).abs().max().item() < tol
    refb = torch.relu(_ref(a, b, None, None))
    assert (outb.float() - refb).abs().max().item() < 3e-2 * max(1.0, refb.abs().max().item())


def _mk32(rows, cols, mn_major, scale=1.0):
    """fp32 [rows(MN), cols(K)] view, stored K-major or MN-major."""
    if mn_major:
        return (torch.randn(cols, rows, device="cuda") * scale).t()
    return torch.randn(rows, cols, device="cuda") * scale


@pytest.mark.parametrize("kernel", ["1cta", "2cta"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1), (1, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (128, 128, 96), (256, 512, 512), (384, 200, 328), (136, 72, 1000),
                                   (1024, 1000, 2048)])
def test_gemm_tf32_layouts(a_mn, b_mn, M, N, K, kernel):
    """fp32 operands on the tensor cores (tcgen05 kind::tf32) against a float64 product."""
    from ferrum_b200.ops.gemm import gemm_tf32
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(M * 5 + N * 3 + K + a_mn * 2 + b_mn)
    a = _mk32(M, K, a_mn, 0.5)
    b = _mk32(N, K, b_mn, 0.5)
    out = gemm_tf32(a, b, kernel=kernel)
    check_status()
    # The tensor core reads 10 mantissa bits of each fp32 operand; whether the rest is cut or rounded is the
    # hardware's choice, so the sharp comparison takes the closer of the two emulations (float64 products of the
    # reduced operands), and a loose one bounds the distance to the exact product.
    def emul(rnd):
        ar = (a.contiguous().view(torch.int32) + (0x1000 if rnd else 0)) & ~0x1FFF
        br = (b.contiguous().view(torch.int32) + (0x1000 if rnd else 0)) & ~0x1FFF
        return (ar.view(torch.float32).double() @ br.view(torch.float32).double().t()).float()

    exact = (a.double() @ b.double().t()).float()
    e_cut = (out - emul(False)).abs().max().item()
    e_rnd = (out - emul(True)).abs().max().item()
    e_exact = (out - exact).abs().max().item()
    msg = f"{kernel} {M}x{N}x{K} a_mn={a_mn} b_mn={b_mn}: cut {e_cut:.3e} round {e_rnd:.3e} exact {e_exact:.3e}"
    assert min(e_cut, e_rnd) < 2e-5 * K ** 0.5 + 2e-5, msg
    assert e_exact < 1e-3 * K ** 0.5 + 1e-3, msg


def test_gemm_tf32_epilogue_and_accumulate():
    from ferrum_b200.ops.gemm import gemm_tf32

    torch.manual_seed(3)
    M, N, K = 300, 520, 192
    a, b = _mk32(M, K, 0, 0.3), _mk32(N, K, 0, 0.3)
    bias = torch.randn(N, device="cuda")
    out = gemm_tf32(a, b, bias=bias, act="gelu")
    ref = _ref(a, b, bias, "gelu")
    assert (out - ref).abs().max().item() < 5e-3
    acc = torch.ones(M, N, device="cuda")
    gemm_tf32(a, b, out=acc, accumulate=True)
    assert (acc - (1.0 + _ref(a, b, None, None))).abs().max().item() < 5e-3


def test_tf32_precision_mode_trains_a_linear_layer():
    import ferrum_b200 as fb
    from ferrum_b200 import _lib, nn

    torch.manual_seed(4)
    dev = fb.Device.Cuda(0)
    lin = nn.Linear(128, 64, device=dev)
    x = torch.randn(96, 128, device="cuda", requires_grad=True)
    prev = fb.config.matmul_precision()
    fb.config.matmul_precision("tf32")
    try:
        before = _lib.launch_count()
        y = lin(x)
        y.square().mean().backward()
        assert _lib.launch_count() > before and y.dtype == torch.float32
    finally:
        fb.config.matmul_precision(prev)
    xr = x.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr, lin.weight.detach(), lin.bias.detach())
    yr.square().mean().backward()
    assert (y - yr).abs().max().item() < 5e-3
    assert (x.grad - xr.grad).abs().max().item() < 1e-4 + 5e-3 * xr.grad.abs().max().item()


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 512), (2560, 1000, 192), (776, 264, 136)])
def test_cta_pair_gemm_store_paths(M, N, K):
    """The three ways a result leaves the CTA-pair kernel: slabs through the TMA unit (store, and reduce-add when
    accumulating), both outputs of the value + derivative epilogue, and register stores for a result whose row
    pitch the TMA unit cannot address (an odd-pitched view).  Run twice so that slab reuse across launches shows."""
    from ferrum_b200.ops.gemm import gemm_bf16
    from ferrum_b200.utils.runtime import check_status

    torch.manual_seed(M + N + K)
    a = (torch.randn(K, M, device="cuda") * 0.5).bfloat16().t()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda")
    ref = a.double() @ b.double().t()
    tol = 2e-3 * K ** 0.5 * 0.25 + 1e-3
    for _ in range(2):
        out = torch.full((M, N), 2.0, device="cuda")
        gemm_bf16(a, b, out=out, accumulate=True)
        assert (out.double() - (ref + 2.0)).abs().max().item() < tol
        # odd pitch: columns 1 .. N of a wider matrix (base and pitch off the 16-byte grid); neighbours stay untouched
        wide = torch.full((M, N + 3), -7.0, device="cuda")
        gemm_bf16(a, b, bias=bias, out=wide[:, 1:N + 1])
        assert (wide[:, 1:N + 1].double() - (ref + bias)).abs().max().item() < tol
        assert (wide[:, 0] == -7.0).all() and (wide[:, N + 1:] == -7.0).all()
        wide_b = torch.full((M, N + 3), -7.0, device="cuda", dtype=torch.bfloat16)
        gemm_bf16(a, b, bias=bias, act="relu", out=wide_b[:, 1:N + 1])
        want = torch.relu(ref + bias)
        assert (wide_b[:, 1:N + 1].double() - want).abs().max().item() < 3e-2 * max(1.0, want.abs().max().item())
        assert (wide_b[:, 0] == -7.0).all() and (wide_b[:, N + 1:] == -7.0).all()
        # TMA path next to memory that must stay untouched: a [M, N] block inside a wider 16-byte-pitched matrix
        pad = (-N) % 8 + 8
        host = torch.full((M + 2, N + pad), 5.0, device="cuda", dtype=torch.bfloat16)
        der = torch.full((M + 2, N + pad), 5.0, device="cuda", dtype=torch.bfloat16)
        gemm_bf16(a, b, bias=bias, act="gelu", out=host[1:M + 1, :N], act_grad=der[1:M + 1, :N])
        z = (ref + bias).float().requires_grad_(True)
        val = torch.nn.functional.gelu(z, approximate="tanh")
        val.sum().backward()
        assert (host[1:M + 1, :N].float() - val).abs().max().item() < 3e-2 * max(1.0, val.abs().max().item())
        assert (der[1:M + 1, :N].float() - z.grad).abs().max().item() < 2e-2
        for t in (host, der):
            assert (t[0] == 5.0).all() and (t[M + 1] == 5.0).all() and (t[:, N:] == 5.0).all()
        check_status()
