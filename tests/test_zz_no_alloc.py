"""Decode through the entry point that brings its own scratch memory.

``rq_decode_static_scratch`` serves callers that cannot give ``rq_decode`` a workspace because
they have no device memory to spare or are not allowed to allocate when the call is made (a
server whose HBM is already committed to its KV-cache pool, a runtime that bans allocator calls
on its request path).  The test drives it through the C ABI with raw pointers, twice in a row on
the shared scratch area, and checks both results against the regular entry point.  It is
collected last so that a failure here cannot hide the result of any other test.
"""

import math

import pytest
import torch

import gpu_util
from gpu_util import DEV
from oracle import rq_oracle, tolerance
from rotorquant_vllm import _lib
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu

STATIC_BYTES = 16 << 20


def _case(lens, seed):
    p = gpu_util.params("iso_fast", 3, 3)
    H, HQ, bs = 8, 32, 16
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, seed)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, torch.bfloat16, seed)
    cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, cache, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    q = syn.make_queries(len(lens), HQ, 128, torch.bfloat16, seed)
    return {k: v.to(DEV) for k, v in dict(q=q, cache=cache, bt=bt, sl=seq_lens, ck=p["k_centroids"],
                                          cv=p["v_centroids"], R=p["R"]).items()}, H, HQ, bs


def _call(fn_name, c, H, HQ, bs, out, workspace=None):
    L = _lib.lib()
    q = c["q"]
    common = (q.data_ptr(), out.data_ptr(), _lib.dtype_code(q.dtype), q.stride(0), q.stride(1),
              out.stride(0), out.stride(1), q.shape[0], HQ, H, 128, c["cache"].data_ptr(),
              c["cache"].shape[0], bs, c["cache"].shape[2], c["bt"].data_ptr(), c["bt"].stride(0),
              c["sl"].data_ptr(), c["ck"].data_ptr(), c["ck"].numel(), c["cv"].data_ptr(),
              c["cv"].numel(), c["R"].data_ptr(), 1.0 / math.sqrt(128), c["bt"].shape[1] * bs)
    stream = torch.cuda.current_stream().cuda_stream
    if workspace is None:
        return getattr(L, fn_name)(*common, 0, stream)
    return getattr(L, fn_name)(*common, workspace.data_ptr(), workspace.numel(), 0, stream)


def test_static_scratch_decode_matches_regular_decode_twice():
    torch.cuda.set_device(DEV)
    for lens, seed in (([700, 33, 1, 260], 21), ([4096, 17], 22)):      # second call reuses the area
        c, H, HQ, bs = _case(lens, seed)
        want = torch.empty_like(c["q"])
        ws = torch.empty(STATIC_BYTES, dtype=torch.uint8, device=DEV)
        assert _call("rq_decode", c, H, HQ, bs, want, workspace=ws) == 0
        got = torch.full_like(c["q"], 9.0)
        status = _call("rq_decode_static_scratch", c, H, HQ, bs, got)
        assert status == 0, _lib.lib().rq_last_error()
        torch.cuda.synchronize()
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2e-3, diff
        assert not bool(torch.isnan(got.float()).any())
        # and against the oracle, so that a fault shared by both entry points cannot pass
        p = gpu_util.params("iso_fast", 3, 3)
        args = (c["q"].cpu(), c["cache"].cpu(), c["bt"].cpu(), c["sl"].cpu(), p["k_centroids"], p["v_centroids"],
                p["R"], H, 128, bs)
        worst, over = tolerance.excess(got.cpu(), rq_oracle.decode(*args, return_rotated_fp32=True),
                                       rq_oracle.decode(*args), torch.bfloat16)
        assert over == 0, (worst, over)


def test_static_scratch_rejects_oversized_calls():
    """A call that needs more scratch than the built-in area is refused before any launch."""
    L = _lib.lib()
    need = L.rq_decode_workspace_bytes(4096, 32, 8, 128, 8192, 0)
    assert need > STATIC_BYTES
    status = L.rq_decode_static_scratch(16, 16, 2, 4096, 128, 4096, 128, 4096, 32, 8, 128, 16, 8, 16, 2048,
                                        16, 8, 16, 16, 8, 16, 8, 16, 0.088, 8192, 0, None)
    assert status == _lib.RQ_ERR_WORKSPACE
    assert b"built-in area" in L.rq_last_error()
