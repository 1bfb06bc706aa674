"""The allocation-free entry point gsq_linear_vec_static against the ordinary two-call path.

Some hosts of this library cannot allocate device memory at the moment they need a product (their own
memory manager holds the whole device, or they only receive input / output pointers), so the library keeps
the intermediate q8_1 blocks in a fixed array of its own. This checks, through the C ABI, that it gives
exactly what gsq_quantize_q8_1 + gsq_mul_mat_vec_q8 give with a caller-owned buffer -- on two calls in a
row with different inputs, since the array is shared and keeps the previous call's bytes -- and that shapes
beyond the array are refused. Collected last so that a failure here cannot hide another test's result.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _both(lib, w, t, packed, x, rows):
    m, k = x.shape
    st = torch.cuda.current_stream().cuda_stream
    y_static = torch.empty(m, rows, dtype=x.dtype, device=DEV)
    rc = lib.gsq_linear_vec_static(w.data_ptr(), w.shape[1], rows, t, int(packed), x.data_ptr(), DT[x.dtype], m, k,
                                   x.stride(0), y_static.data_ptr(), DT[x.dtype], rows, st)
    assert rc == 0, lib.gsq_strerror(rc)
    xq = torch.empty(m * k // 32 * 36, dtype=torch.uint8, device=DEV)
    y_ref = torch.empty(m, rows, dtype=x.dtype, device=DEV)
    assert lib.gsq_quantize_q8_1(x.data_ptr(), DT[x.dtype], m, k, x.stride(0), xq.data_ptr(), st) == 0
    assert lib.gsq_mul_mat_vec_q8(w.data_ptr(), w.shape[1], rows, t, int(packed), xq.data_ptr(), m, k,
                                  y_ref.data_ptr(), DT[x.dtype], rows, st) == 0
    torch.cuda.synchronize()
    return y_static, y_ref


@pytest.mark.parametrize("name,t,packed", [("IQ3_S", 21, True), ("Q4_K", 12, False)])
def test_static_scratch_matches_two_call_path_twice(name, t, packed):
    from gsq_b200 import _cabi, synth
    from gsq_b200.quantization import iq3_pack

    lib = _cabi.lib
    rows, k = 272, 5120
    w = torch.from_numpy(synth.make_weight(t, rows, k, 3)).to(DEV)
    if packed:
        iq3_pack.pack_(w, t)
    # first call: 8 rows fill the array; second call: 3 other rows reuse its beginning
    for m, seed, dtype in ((8, 10, torch.float16), (3, 11, torch.bfloat16)):
        x = torch.from_numpy(synth.make_activation(m, k, seed)).to(dtype).to(DEV)
        y_static, y_ref = _both(lib, w, t, packed, x, rows)
        assert torch.equal(y_static, y_ref)          # same kernels, same bytes: bit identical
        assert torch.isfinite(y_static.float()).all() and float(y_static.float().abs().max()) > 0


def test_static_entry_point_allocates_nothing():
    """After one warm-up call (which resolves the array's address) the free device memory reported by the driver
    is the same before and after a call, and a bad weight type is refused before anything is launched."""
    from gsq_b200 import _cabi, synth

    lib = _cabi.lib
    rows, k, m = 64, 1024, 4
    w = torch.from_numpy(synth.make_weight(12, rows, k, 5)).to(DEV)
    x = torch.from_numpy(synth.make_activation(m, k, 6)).to(torch.float16).to(DEV)
    y = torch.empty(m, rows, dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream

    def call(t=12):
        return lib.gsq_linear_vec_static(w.data_ptr(), w.shape[1], rows, t, 0, x.data_ptr(), 1, m, k, k, y.data_ptr(), 1,
                                         rows, st)
    assert call() == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert call(t=2) == _cabi.ERR_UNSUPPORTED          # not a type with a kernel: refused, nothing queued


def test_static_scratch_rejects_what_does_not_fit():
    from gsq_b200 import _cabi

    lib = _cabi.lib
    assert lib.gsq_linear_vec_static_max_q8_bytes() == 8 * (32768 // 32) * 36
    w = torch.zeros(16, 144 * 2, dtype=torch.uint8, device=DEV)
    x = torch.zeros(9, 512, dtype=torch.float16, device=DEV)
    y = torch.zeros(9, 16, dtype=torch.float16, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.gsq_linear_vec_static(w.data_ptr(), 288, 16, 12, 0, x.data_ptr(), 1, 9, 512, 512, y.data_ptr(), 1, 16, st)
    assert rc == _cabi.ERR_TOO_LARGE and b"too large" in lib.gsq_strerror(rc)
    # 8 rows of 65536 columns would need twice the array
    rc = lib.gsq_linear_vec_static(w.data_ptr(), 144 * 256, 16, 12, 0, x.data_ptr(), 1, 8, 65536, 65536, y.data_ptr(), 1,
                                   16, st)
    assert rc == _cabi.ERR_TOO_LARGE
