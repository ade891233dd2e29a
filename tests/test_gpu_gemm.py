"""tcgen05 GEMM against an fp32 PyTorch reference (one GPU)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(got, ref):
    return (got.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)


@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 128), (384, 768, 320),
                                   (1000, 520, 136), (2048, 2048, 1024), (130, 264, 72)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_gemm_matches_fp32_reference(shape, dtype, b_is_nk):
    from tileccl_b200.kernels.fused_gemm import gemm

    M, N, K = shape
    torch.manual_seed(M + N + K)
    a = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dtype)
    b = torch.randn(K, N, device="cuda").to(dtype)
    c = gemm(a, b.t().contiguous() if b_is_nk else b, b_is_nk=b_is_nk)
    torch.cuda.synchronize()
    assert _rel_err(c, a.float() @ b.float()) < (2e-2 if dtype is torch.bfloat16 else 4e-3)


def test_silu_gate_epilogue():
    from tileccl_b200.kernels.fused_gemm import gemm
    from tileccl_b200.models import pack_gate_up

    M, K, F = 512, 256, 512
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") / K ** 0.5).bfloat16()
    wg = (torch.randn(K, F, device="cuda")).bfloat16()
    wu = (torch.randn(K, F, device="cuda")).bfloat16()
    out = gemm(x, pack_gate_up(wg, wu), epilogue="silu_gate")
    ref = torch.nn.functional.silu(x.float() @ wg.float()) * (x.float() @ wu.float())
    assert out.shape == (M, F) and _rel_err(out, ref) < 3e-2


def test_strided_views_and_repeat_calls():
    from tileccl_b200.kernels.fused_gemm import gemm

    torch.manual_seed(1)
    big_a = (torch.randn(512, 512, device="cuda") / 16).half()
    big_b = torch.randn(512, 1024, device="cuda").half()
    a, b = big_a[:, :256], big_b[:256, 256:768]          # row pitch != width
    out = torch.zeros(512, 1024, device="cuda", dtype=torch.float16)
    c = out[:, 128:640]
    for _ in range(3):
        gemm(a, b, c)
    torch.cuda.synchronize()
    assert _rel_err(c, a.float() @ b.float()) < 4e-3
    assert out[:, :128].abs().max() == 0 and out[:, 640:].abs().max() == 0   # nothing outside the view


def test_argument_errors():
    from tileccl_b200 import _native
    from tileccl_b200.kernels.fused_gemm import gemm

    a = torch.randn(128, 64, device="cuda").half()
    with pytest.raises(ValueError):
        gemm(a, torch.randn(32, 128, device="cuda").half())
    with pytest.raises(TypeError):
        gemm(a.float(), torch.randn(64, 128, device="cuda"))
    with pytest.raises(TypeError):
        gemm(a, torch.randn(64, 128, device="cuda").bfloat16())
    with pytest.raises(_native.NativeError):             # K not a multiple of 8 elements
        gemm(torch.randn(128, 60, device="cuda").half(), torch.randn(60, 128, device="cuda").half())


@pytest.mark.parametrize("b_is_nk", [False, True])
def test_one_cta_and_cta_pair_kernels_agree(monkeypatch, b_is_nk):
    """The plain GEMM runs on CTA pairs by default; TILECCL_GEMM_2SM=0 keeps the one-CTA
    kernel.  Same inputs, same fp32 accumulation order inside a tile: identical output."""
    from tileccl_b200.kernels import fused_gemm as fg

    M, N, K = 896, 768, 448          # 7 tile rows: the last pair has one real half
    torch.manual_seed(5)
    a = (torch.randn(M, K, device="cuda") / K ** 0.5).half()
    b = torch.randn(K, N, device="cuda").half()
    bb = b.t().contiguous() if b_is_nk else b
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("TILECCL_GEMM_2SM", flag)
        c = torch.zeros(M, N, device="cuda", dtype=torch.float16)
        spec = fg.FusedGemmSpec(
            mode=fg.MODE_GEMM, dtype=torch.float16, a_ptr=a.data_ptr(), a_rows=M, lda=K,
            b_ptr=bb.data_ptr(), b_cols=N, ldb=bb.stride(0), k=K, sub_m=M, sub_n=N,
            out_ptrs=[c.data_ptr()], ldo=N, out_rows=M, out_cols=N, b_kmajor=b_is_nk)
        plan = fg.FusedGemmPlan(spec)
        plan.launch()
        torch.cuda.synchronize()
        plan.close()
        outs.append(c)
    assert _rel_err(outs[0], a.float() @ b.float()) < 4e-3
    assert torch.equal(outs[0], outs[1])
