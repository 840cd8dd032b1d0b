"""The allocation-free panel entry point against the regular one.

Some callers cannot allocate device memory at the moment they need a panel factored (they are
inside a stream capture, or a host framework owns all device memory, or they must not block on the
allocator).  For them the library exports one C symbol, ``soapb200_qr_panel_noalloc``, whose
exchange scratch is a fixed array inside the library.  This test calls that symbol through
``ctypes`` twice in a row -- the second time on a smaller panel, so the array still holds the first
call's words -- and checks every output against the regular entry point, which uses a scratch
buffer supplied by the caller.  It also checks that an oversized panel is refused with a message.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from soap_tp_b200.engine import kernels as k

    library = ctypes.CDLL(k._C.__file__)
    entry = library.soapb200_qr_panel_noalloc
    entry.restype = ctypes.c_int
    entry.argtypes = ([ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p,
                       ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                       ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p,
                       ctypes.c_int])
    return k, entry


class _Outputs:
    def __init__(self, k, rows, cols):
        self.v = k.Planes.empty(rows, cols, "cuda")
        self.vt = k.Planes.empty(cols, rows, "cuda")
        self.t = k.Planes.empty(cols, cols, "cuda")
        self.tt = k.Planes.empty(cols, cols, "cuda")
        self.tau = torch.zeros(cols, device="cuda")
        for planes in (self.v, self.vt, self.t, self.tt):
            planes.hi.zero_()
            planes.lo.zero_()

    def tensors(self):
        return [self.v.hi, self.v.lo, self.vt.hi, self.vt.lo, self.t.hi, self.t.lo, self.tt.hi, self.tt.lo, self.tau]


def _factor_both(k, entry, rows, cols, seed):
    generator = torch.Generator(device="cuda").manual_seed(seed)
    panel = k.split_planes(torch.randn(rows, cols, generator=generator, device="cuda"))
    status = k.status_word(torch.device("cuda", torch.cuda.current_device()))
    stream = torch.cuda.current_stream().cuda_stream

    regular = _Outputs(k, rows, cols)
    exchange = torch.zeros(4 * (rows // 256 + 2) * 128 + 512, dtype=torch.float32, device="cuda")
    k._C.qr_panel(panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, rows, cols, regular.v.hi.data_ptr(),
                  regular.v.lo.data_ptr(), regular.v.ld, regular.vt.hi.data_ptr(), regular.vt.lo.data_ptr(), regular.vt.ld,
                  regular.tau.data_ptr(), regular.t.hi.data_ptr(), regular.t.lo.data_ptr(), regular.tt.hi.data_ptr(),
                  regular.tt.lo.data_ptr(), regular.t.ld, exchange.data_ptr(), status.data_ptr(), stream)

    fixed = _Outputs(k, rows, cols)
    message = ctypes.create_string_buffer(256)
    code = entry(panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, rows, cols, fixed.v.hi.data_ptr(),
                 fixed.v.lo.data_ptr(), fixed.v.ld, fixed.vt.hi.data_ptr(), fixed.vt.lo.data_ptr(), fixed.vt.ld,
                 fixed.tau.data_ptr(), fixed.t.hi.data_ptr(), fixed.t.lo.data_ptr(), fixed.tt.hi.data_ptr(),
                 fixed.tt.lo.data_ptr(), fixed.t.ld, status.data_ptr(), stream, message, 256)
    assert code == 0, message.value.decode()
    torch.cuda.synchronize()
    k.check_status()
    for got, want in zip(fixed.tensors(), regular.tensors()):
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    # the factorisation itself is sound: V has a unit diagonal and tau is in [0, 2]
    dense_v = fixed.v.dense()
    assert torch.allclose(torch.diagonal(dense_v)[: min(rows, cols)], torch.ones(min(rows, cols), device="cuda"))
    assert float(fixed.tau.min()) >= 0.0 and float(fixed.tau.max()) <= 2.0


def test_no_alloc_entry_point_matches_regular_entry_point_twice():
    k, entry = _load()
    _factor_both(k, entry, 1500, 128, seed=1)     # six thread blocks exchange through the built-in scratch
    _factor_both(k, entry, 700, 96, seed=2)       # second call: fewer blocks, the scratch holds stale words


def test_no_alloc_entry_point_at_its_documented_maximum():
    """16384 rows x 128 columns: 64 thread blocks, every word of the built-in scratch is in use."""
    k, entry = _load()
    _factor_both(k, entry, 16384, 128, seed=3)
    _factor_both(k, entry, 16384, 128, seed=4)    # again, over the previous call's words


def test_no_alloc_entry_point_on_a_second_device():
    """The scratch address is resolved per device, and the kernel's shared-memory limit is raised per device."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    k, entry = _load()
    with torch.cuda.device(1):
        _factor_both_on = lambda: _factor_both(k, entry, 1500, 128, seed=5)
        # tensors created with device="cuda" follow the current device
        _factor_both_on()
        _factor_both_on()


def test_no_alloc_entry_point_refuses_oversized_panels():
    k, entry = _load()
    dummy = torch.zeros(8, device="cuda")
    status = k.status_word(torch.device("cuda", torch.cuda.current_device()))
    message = ctypes.create_string_buffer(256)
    pointers = [dummy.data_ptr()] * 2
    code = entry(*pointers, 4, 20000, 128, *pointers, 4, *pointers, 4, dummy.data_ptr(), *pointers, *pointers, 4,
                 status.data_ptr(), None, message, 256)
    assert code != 0 and b"exceeds" in message.value
    code = entry(*pointers, 4, 256, 200, *pointers, 4, *pointers, 4, dummy.data_ptr(), *pointers, *pointers, 4,
                 status.data_ptr(), None, message, 256)
    assert code != 0 and b"exceeds" in message.value
