"""The allocation-free attention entry (lrqk_flash_decode_static) against the ordinary one.

Some hosts of this library cannot allocate device memory when they call it -- their runtime has
already given every byte to its own pool, or their rules forbid allocator calls in the step --
so they cannot supply the workspace lrqk_flash_decode needs.  The static entry keeps its scratch
in an array inside the library instead.  Both entries run the same kernel, so their outputs must
agree bit for bit; the test calls the static entry twice in a row (the array keeps the previous
call's contents) and also checks the size limit.  It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_matches_workspace_attention():
    from lrqk_b200 import _lib
    from lrqk_b200.state import LayerState
    lib = _lib.lib()
    stream = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.lrqk_flash_decode_static_capacity_bytes() == 4 << 20
    g = torch.Generator().manual_seed(123)
    for dtype, bsz, hq, rows in ((torch.bfloat16, 1, 32, 2112), (torch.float32, 2, 8, 272)):
        st = LayerState(bsz, hq, hq, 128, 16, rows - 8, 8, a_capacity=64, host_capacity=16, dtype=dtype,
                        with_host=False)
        st.K_res.copy_(torch.randn(bsz, hq, rows, 128, generator=g).to(dtype))
        st.V_res.copy_(torch.randn(bsz, hq, rows, 128, generator=g).to(dtype))
        out = torch.empty(bsz, hq, 128, dtype=dtype, device="cuda")
        for call in range(2):                      # two calls in a row on the shared array
            q = torch.randn(bsz, hq, 128, generator=g).to(dtype).cuda()
            ref = st.flash_decode(q).clone()
            out.fill_(float("nan"))
            _lib.check(lib.lrqk_flash_decode_static(C.byref(st.c), C.c_void_p(q.data_ptr()),
                                                    C.c_void_p(out.data_ptr()), rows, 128 ** -0.5, stream()),
                       "lrqk_flash_decode_static")
            status = torch.full((1,), -99, dtype=torch.int32).pin_memory()
            _lib.check(lib.lrqk_flash_decode_static_status(C.c_void_p(status.data_ptr()), stream()),
                       "lrqk_flash_decode_static_status")
            torch.cuda.synchronize()
            assert torch.equal(out, ref), f"{dtype} call {call}"
            assert int(status[0]) == 0                 # no bounded wait of the call ran out
    # beyond the built-in array: a clear refusal, nothing launched
    big = LayerState(128, 64, 64, 128, 16, 24, 8, a_capacity=64, host_capacity=16, dtype=torch.bfloat16,
                     with_host=False)                       # 8192 heads x 520 bytes > 4 MiB
    q = torch.zeros(128, 64, 128, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros_like(q)
    rc = lib.lrqk_flash_decode_static(C.byref(big.c), C.c_void_p(q.data_ptr()), C.c_void_p(o.data_ptr()), 32,
                                      0.1, stream())
    assert rc == _lib.ECAPACITY
    assert b"built-in array" in lib.lrqk_last_cuda_error()
