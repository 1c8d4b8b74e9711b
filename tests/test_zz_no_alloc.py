"""The decode attention entry point that allocates nothing, called through its
exported C symbol as a host without an allocator would call it.

It serves programs that plan all device memory ahead and may not allocate later
(a serving loop with a fixed memory plan, a plug-in that is handed buffers but
no allocator): the scratch between the kernel's two passes is a static array in
the library.  The test checks its output against the ordinary entry point, whose
scratch the caller allocates, on two calls in a row, and that a request beyond
the array's size is refused.  This file is collected last on purpose, so that a
run that stops at the first failure has already run every other test.
"""

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

from test_gpu_kernels import paged_case, paged_reference

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _symbols(head_dim):
    from inf_engine_b200 import kernels
    path = kernels.attention_mma_library(head_dim)._path
    lib = ctypes.CDLL(path)                      # the exported C symbols, as any host program sees them
    P, I, F = c_void_p, c_int, c_float
    lib.ie_attention_decode_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P]
    lib.ie_attention_decode_noalloc.restype = c_int
    lib.ie_attention_decode.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P]
    lib.ie_attention_decode.restype = c_int
    lib.ie_attention_decode_noalloc_capacity.restype = c_longlong
    lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
    lib.ie_attention_decode_scratch_floats.restype = c_longlong
    return lib


# the second case has one request of 3,500 keys cut into 55 splits: more blocks per (request, kv head) than a cluster
# holds, so the blocks add up through the static array (partial results and a ticket per request and kv head) and
# the second call finds the first call's partial results there and needs the tickets back at zero
@pytest.mark.parametrize("q_lens,ctx_before", [([1, 1, 2, 1], [700, 33, 250, 0]), ([1, 1], [3500, 40])])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_no_alloc_entry_point_matches_the_ordinary_one(head_dim, q_lens, ctx_before):
    lib = _symbols(head_dim)
    H, Hk, ps, split_keys = 8, 2, 16, 64
    lib.ie_attention_decode_warps.restype = c_int
    if max(ctx_before) > 3000:
        assert -(-(max(ctx_before) + 1) // split_keys) > 8 * lib.ie_attention_decode_warps()    # the ticket path
    bf = torch.bfloat16
    dev = lambda t: torch.as_tensor(t, dtype=torch.int32).to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                         # two calls in a row share the static array
        c = paged_case(bf, H, Hk, head_dim, ps, q_lens, ctx_before, seed=40 + call)
        ref = paged_reference(c["q"], c["kd"], c["vd"], q_lens, ctx_before, H, Hk, head_dim, None)
        q, kp, vp = c["q"].to(DEV, bf), c["kpool"].to(DEV, bf), c["vpool"].to(DEV, bf)
        table, q_start, ctx = c["table"].to(DEV), dev(c["q_start"]), dev(ctx_before)
        n_splits = -(-(max(a + b for a, b in zip(q_lens, ctx_before))) // split_keys)
        need = lib.ie_attention_decode_scratch_floats(c["N"], H, n_splits)
        assert need <= lib.ie_attention_decode_noalloc_capacity()
        out_a = torch.full((c["N"], H * head_dim), float("nan"), device=DEV, dtype=bf)
        out_b = torch.full_like(out_a, float("nan"))
        scratch = torch.zeros(need, device=DEV)      # the ordinary entry point wants its tickets zeroed by the caller
        common = (q.stride(0), out_a.stride(0), table.stride(0), len(q_lens), c["N"], H, Hk, head_dim, ps, 0,
                  head_dim ** -0.5, n_splits, split_keys, stream)
        rc = lib.ie_attention_decode(q.data_ptr(), out_a.data_ptr(), kp.data_ptr(), vp.data_ptr(), table.data_ptr(),
                                     q_start.data_ptr(), ctx.data_ptr(), scratch.data_ptr(), *common)
        assert rc == 0
        rc = lib.ie_attention_decode_noalloc(q.data_ptr(), out_b.data_ptr(), kp.data_ptr(), vp.data_ptr(),
                                             table.data_ptr(), q_start.data_ptr(), ctx.data_ptr(), *common)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(out_a, out_b)          # same kernels, same order of sums
        assert torch.allclose(out_b.float().cpu(), ref, atol=2e-2, rtol=2e-2)


def test_no_alloc_entry_point_refuses_more_than_its_array_holds():
    lib = _symbols(64)
    cap = lib.ie_attention_decode_noalloc_capacity()
    assert cap == 1 << 20
    n_tokens, H, n_splits = 64, 32, 64            # 64*32*64*66 floats: far beyond the array
    assert n_tokens * H * n_splits * 66 > cap
    z = torch.zeros(16, device=DEV, dtype=torch.bfloat16)
    zi = torch.zeros(80, device=DEV, dtype=torch.int32)
    rc = lib.ie_attention_decode_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), zi.data_ptr(),
                                         zi.data_ptr(), zi.data_ptr(), 64, 64, 1, 64, n_tokens, H, 8, 64, 16, 0, 1.0,
                                         n_splits, 32, torch.cuda.current_stream().cuda_stream)
    assert rc == -4                                # IE_NOALLOC_TOO_LARGE: nothing was launched
