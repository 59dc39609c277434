"""The tcgen05 GEMM engine alone (lce_debug_gemm): every operand layout of the three contractions, for each
input type, against a float64 product."""
import pytest
import torch

from linear_cross_entropy_loss_b200 import _native

pytestmark = pytest.mark.gpu

CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


SINGLE_CTA = 0


@pytest.fixture(params=[0, 1], ids=["cta_pair", "single_cta"], autouse=True)
def gemm_variant(request):
    """Every test of this file runs once per kernel variant (pair kernels need M % 256 == 0, else fall back)."""
    global SINGLE_CTA
    SINGLE_CTA = request.param
    yield request.param
    SINGLE_CTA = 0


def run(dtype, a_mn, b_mn, M, N, K, splits=1, seed=0, raster_group=0, n_fastest=0):
    lib = _native.load()
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(dtype)
    B = torch.randn(N, K, generator=g).to(dtype)
    ref = A.double() @ B.double().T
    a = (A.T.contiguous() if a_mn else A).cuda()
    b = (B.T.contiguous() if b_mn else B).cuda()
    out = torch.full((splits, M, N), float("nan"), dtype=torch.float32, device="cuda")
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.lce_debug_gemm(CODE[dtype], a_mn, b_mn, a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                            out.data_ptr(), M, N, K, splits, SINGLE_CTA, raster_group, n_fastest, status.data_ptr(),
                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.status_string(rc)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    got = out.double().sum(0).cpu()
    return (got - ref).abs().max().item() / ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 1), (0, 0), (1, 1), (1, 0)])
def test_all_operand_layouts(dtype, a_mn, b_mn):
    # (0,1) logits z = x W, (0,0) dx = dZ W^T, (1,1) dW = x^T dZ
    tol = 2e-3 if dtype == torch.float32 else 1e-5   # TF32 keeps 10 mantissa bits of each input
    assert run(dtype, a_mn, b_mn, 256, 512, 512) < tol


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_split_k_partials_sum_to_the_product(dtype):
    tol = 2e-3 if dtype == torch.float32 else 1e-5
    assert run(dtype, 0, 0, 256, 256, 4096, splits=4) < tol


def test_more_tiles_than_sms_and_long_k():
    assert run(torch.bfloat16, 0, 1, 128 * 23, 256 * 9, 256) < 1e-5     # 207 tiles: several per CTA
    assert run(torch.float16, 1, 1, 128, 256, 64 * 150) < 1e-4           # 150 K-blocks through a 4-deep ring
    #                                                                      (fp32 accumulation over K = 9600)


@pytest.mark.parametrize("n_fastest", [0, 1])
@pytest.mark.parametrize("group", [1, 2, 3, 5, 64])
def test_banded_walk_over_the_tile_grid_visits_every_tile_once(group, n_fastest):
    # 11 x 7 tiles of 128 x 256 (single CTA) or 5 x 7 of 256 x 256 (CTA pairs), two K splits; bands that do not
    # divide the fast dimension and a band wider than the grid. The output starts as NaN: a tile that no unit
    # visits fails the comparison, and so does one that holds another tile's product.
    m_tiles = 11 if SINGLE_CTA else 10
    assert run(torch.bfloat16, 0, 1, 128 * m_tiles, 256 * 7, 256, splits=2, raster_group=group,
               n_fastest=n_fastest) < 1e-5


def test_shape_errors_are_status_codes():
    lib = _native.load()
    t = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(256, 256, dtype=torch.float32, device="cuda")
    s = torch.zeros(8, dtype=torch.int32, device="cuda")
    call = lambda m, n, k, sp=1: lib.lce_debug_gemm(1, 0, 0, t.data_ptr(), 256, t.data_ptr(), 256, o.data_ptr(), m, n,
                                                    k, sp, SINGLE_CTA, 0, 0, s.data_ptr(), None)
    assert call(100, 256, 256) == -2
    assert call(128, 100, 256) == -2
    assert call(128, 256, 100) == -2
    assert call(128, 256, 256, 3) == -2
