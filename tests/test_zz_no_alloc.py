"""The allocation-free routing entry point (moe_fp8_b200_route_noalloc), called through the
C ABI, against the regular entry point (moe_fp8_b200_run and its intermediate buffers).

That entry point serves callers that may not allocate device memory where they need the
routing result (frozen memory pools, serving loops, hosts that forbid library-side
cudaMalloc); its scratch is a fixed array inside the library that every call shares.  The
test therefore makes two calls in a row with different inputs and sizes: the second must
not see anything of the first (counters are cleared per call), and both must agree bit for
bit with what the regular path computes.  The file sorts last so that a run that stops at
the first failure has already been through every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import helpers as hp
from helpers import TOPK

pytestmark = pytest.mark.gpu


def route_noalloc(pkg, logits, bias, offset, E, rsf, pruning=True):
    lib = pkg._lib.load()
    T = logits.shape[0]
    idx = torch.full((max(T, 1), TOPK), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros(max(T, 1), TOPK, dtype=torch.float32, device="cuda")
    cnt = torch.full((E,), -1, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.moe_fp8_b200_route_noalloc(logits.data_ptr(), bias.data_ptr(), T, offset, E, rsf, int(pruning),
                                        idx.data_ptr(), w.data_ptr(), cnt.data_ptr(), stream, err, len(err))
    return rc, err.value.decode(), idx, w, cnt


def test_two_calls_in_a_row_match_the_regular_entry_point(pkg):
    weights = hp.gpu_shard(0, 32)
    layer = pkg.MoeLayer(1024, 32, 0)
    try:
        # The first call on a GPU does the one-time set-up (the library image with its
        # scratch array is loaded, the array's address is looked up); measure after it.
        warm = hp.cpu_inputs(8, seed=900)
        rc, msg, *_ = route_noalloc(pkg, warm[0].cuda(), warm[1].cuda(), 0, 32, hp.RSF)
        torch.cuda.synchronize()
        assert rc == 0, msg
        for T, offset, seed in ((700, 0, 901), (40, 96, 902)):   # second call is smaller and elsewhere
            inputs = hp.cpu_inputs(T, seed=seed)
            logits, bias = inputs[0].cuda(), inputs[1].cuda()
            free_before = torch.cuda.mem_get_info()[0]
            rc, msg, idx, w, cnt = route_noalloc(pkg, logits, bias, offset, 32, hp.RSF)
            torch.cuda.synchronize()
            assert rc == 0, msg
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the amount of free device memory"
            hp.run_layer(layer, inputs, weights, offset)
            assert np.array_equal(idx.cpu().numpy()[:T], layer.read("topk_idx", T * TOPK).reshape(T, TOPK))
            assert np.array_equal(w.cpu().numpy()[:T].view(np.uint32),
                                  layer.read("topk_weight", T * TOPK).reshape(T, TOPK).view(np.uint32))
            assert np.array_equal(cnt.cpu().numpy(), layer.read("expert_count", 32))
    finally:
        layer.close()


def test_sizes_beyond_the_scratch_are_refused(pkg):
    T = pkg._lib.NOALLOC_MAX_TOKENS + 1
    logits = torch.zeros(T, 256, device="cuda")
    bias = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    rc, msg, _, _, cnt = route_noalloc(pkg, logits, bias, 0, 32, 1.0)
    assert rc == pkg._lib.ERR_CAPACITY and "MOE_FP8_B200_NOALLOC_MAX_TOKENS" in msg
    torch.cuda.synchronize()
    assert int(cnt[0]) == -1, "a refused call must not touch its outputs"
    rc, msg, _, _, _ = route_noalloc(pkg, logits[:8], bias, 0, 48, 1.0)
    assert rc == pkg._lib.ERR_INVALID_ARGUMENT and msg
    # shards are whole blocks of 32 experts inside the 256: an offset between blocks or a block that
    # hangs over the end matches no reference call
    for offset, E in ((16, 32), (240, 32), (224, 64), (-32, 32)):
        rc, msg, _, _, cnt = route_noalloc(pkg, logits[:8], bias, offset, E, 1.0)
        assert rc == pkg._lib.ERR_INVALID_ARGUMENT and "multiple of 32" in msg, (offset, E)
    # host memory is not the current device's memory
    lib = pkg._lib.load()
    host = torch.zeros(8, 256)
    idx = torch.zeros(8, TOPK, dtype=torch.int32, device="cuda")
    w = torch.zeros(8, TOPK, device="cuda")
    cnt = torch.zeros(32, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    rc = lib.moe_fp8_b200_route_noalloc(host.data_ptr(), bias.data_ptr(), 8, 0, 32, 1.0, 1, idx.data_ptr(), w.data_ptr(),
                                        cnt.data_ptr(), torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc == pkg._lib.ERR_INVALID_ARGUMENT and b"current CUDA device" in err.value
