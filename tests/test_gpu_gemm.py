"""The tcgen05 bf16 GEMM and the fp32 CUDA-core GEMM through the C ABI vs a plain PyTorch fp32
reference of the same product (bf16 inputs are exactly representable in fp32, so the only
difference is fp32 summation order)."""
import ctypes

import numpy as np
import pytest
import torch

from cavs_b200 import check, lib

pytestmark = pytest.mark.gpu


def _st():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _run_bf16(cuda, m, n, k, a_major, b_major, out_mode=0, splits=1, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + m * 3 + n * 5 + k * 7)
    A = torch.randn((m, k), generator=g).to(torch.bfloat16)
    B = torch.randn((k, n), generator=g).to(torch.bfloat16)
    ref = A.float().to(cuda) @ B.float().to(cuda)
    a_store = (A if a_major == 0 else A.t()).contiguous().to(cuda)      # [m,k] or [k,m]
    b_store = (B.t() if b_major == 0 else B).contiguous().to(cuda)      # [n,k] or [k,n]
    lda = a_store.shape[1]
    ldb = b_store.shape[1]
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    L = lib()
    L.cavs_gemm_bf16_scratch_bytes.restype = ctypes.c_size_t
    sb = L.cavs_gemm_bf16_scratch_bytes(m, n, splits)
    scratch = torch.empty(max(sb, 4), dtype=torch.uint8, device=cuda)
    if out_mode == 2:
        C = torch.zeros((m, n), dtype=torch.bfloat16, device=cuda)
    else:
        C = torch.ones((m, n), dtype=torch.float32, device=cuda)
    check(L.cavs_gemm_bf16(_p(C), ctypes.c_longlong(n), out_mode, _p(a_store), ctypes.c_longlong(lda), a_major, _p(b_store),
                           ctypes.c_longlong(ldb), b_major, m, n, k, splits, _p(scratch), ctypes.c_size_t(sb), _p(status), _st()))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel expired"
    if out_mode == 1:
        ref = ref + 1.0
    return C.float(), ref


def _check(C, ref, tol, what):
    err = (C - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= tol * scale, f"{what}: max abs err {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("a_major,b_major", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 256, 256), (200, 136, 72), (1000, 3072, 1024), (384, 512, 1032)])
def test_bf16_all_layouts(cuda, a_major, b_major, m, n, k):
    C, ref = _run_bf16(cuda, m, n, k, a_major, b_major)
    _check(C, ref, 2e-5, f"majors {a_major}{b_major} {m}x{n}x{k}")


def test_bf16_accumulate_and_bf16_output(cuda):
    C, ref = _run_bf16(cuda, 300, 256, 512, 0, 1, out_mode=1)
    _check(C, ref, 2e-5, "accumulate")
    C, ref = _run_bf16(cuda, 300, 256, 512, 0, 0, out_mode=2)
    _check(C, ref, 1e-2, "bf16 out")


@pytest.mark.parametrize("splits", [2, 5, 16])
def test_bf16_split_k_weight_gradient_shape(cuda, splits):
    # dW = X^T dY: both operands stored [rows, cols] with the reduction over rows.
    C, ref = _run_bf16(cuda, 256, 512, 5000, 1, 1, splits=splits)
    _check(C, ref, 2e-5, f"split-K {splits}")
    C2, _ = _run_bf16(cuda, 256, 512, 5000, 1, 1, splits=splits)
    assert torch.equal(C, C2), "split-K reduction must be bit-reproducible"


@pytest.mark.parametrize("m,n,k,out_mode", [(1000, 600, 9000, 0), (512, 3072, 20000, 0), (304, 256, 4500, 1)])
def test_bf16_tall_tile_weight_gradients(cuda, m, n, k, out_mode):
    # long-K X^T dY with split-K scratch: the 256 x 256 tile path, with ragged M and N edges and with accumulation
    C, ref = _run_bf16(cuda, m, n, k, 1, 1, splits=4, out_mode=out_mode)
    _check(C, ref, 2e-5, f"tall tiles {m}x{n}x{k} mode {out_mode}")


def test_bf16_tall_tile_deep_k_gradient_product(cuda):
    # dY W^T on a large level: both operands K-major, fp32 out through the TMA-store epilogue, 256 x 256 tiles
    # (ragged last row block)
    C, ref = _run_bf16(cuda, 38000, 1024, 3072, 0, 0)
    _check(C, ref, 2e-5, "tall tiles, deep-K gradient product")


def test_bf16_rejects_misaligned_pitch(cuda):
    from cavs_b200 import CavsError
    with pytest.raises(CavsError):
        A = torch.zeros((8, 12), dtype=torch.bfloat16, device=cuda)
        C = torch.zeros((8, 8), device=cuda)
        check(lib().cavs_gemm_bf16(_p(C), ctypes.c_longlong(8), 0, _p(A), ctypes.c_longlong(12), 0, _p(A), ctypes.c_longlong(12), 0,
                                   8, 8, 12, 1, _p(None), ctypes.c_size_t(0), _p(None), _st()))


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(64, 600, 150), (33, 150, 450), (300, 600, 3264), (1, 5, 7)])
def test_f32_gemm(cuda, ta, tb, m, n, k):
    g = torch.Generator(device="cpu").manual_seed(m + n + k)
    A = torch.randn((m, k), generator=g)
    B = torch.randn((k, n), generator=g)
    ref = (A.double() @ B.double()).float().to(cuda)
    a_store = (A.t() if ta else A).contiguous().to(cuda)
    b_store = (B.t() if tb else B).contiguous().to(cuda)
    a_rs, a_cs = (1, a_store.shape[1]) if ta else (a_store.shape[1], 1)
    b_rs, b_cs = (1, b_store.shape[1]) if tb else (b_store.shape[1], 1)
    C = torch.zeros((m, n), device=cuda)
    ll = ctypes.c_longlong
    check(lib().cavs_gemm_f32(_p(C), ll(n), 0, _p(a_store), ll(a_rs), ll(a_cs), _p(b_store), ll(b_rs), ll(b_cs), m, n, k, _st()))
    torch.cuda.synchronize()
    _check(C, ref, 1e-5, f"f32 gemm {m}x{n}x{k} ta={ta} tb={tb}")
