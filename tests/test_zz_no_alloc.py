"""The no-allocation decode attention (garlic_inference_b200/csrc/no_alloc.h), called through its exported C
symbol the way a host that cannot allocate would call it, against the allocating entry point.

Some callers of this library cannot call cudaMalloc when they need attention (they are inside a stream
capture, or were given a fixed budget and no allocator, or may not block on the allocator's lock), so the
partial results of the key slices go through a fixed array inside the library instead of buffers made per
call.  This file is collected last on purpose: the array is shared by every call in the process, so the
test must hold both alone in a fresh process and after everything else has run."""
import ctypes

import pytest
import torch

from test_gpu_kernels import DEV, K, make_cache

pytestmark = pytest.mark.gpu

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _static_entry():
    from garlic_inference_b200.ops import lib, require_gpu
    require_gpu()
    fn = lib().gi_attention_decode_bf16_static
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
    fn.restype = I
    return fn


def _case(seed, lens, n_q, n_kv, d, page):
    k_pool, v_pool, bt, _, _ = make_cache(len(lens), lens, n_kv, d, page, torch.bfloat16, seed=seed)
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(len(lens), n_q, d, generator=g, device=DEV).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slot = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, bt, pos, slot


def _call_static(fn, q, k_pool, v_pool, bt, pos, slot, scale, window, n_splits):
    n, n_q, d = q.shape
    n_pages, n_kv, page, _ = k_pool.shape
    out = torch.full((n, n_q * d), float("nan"), dtype=torch.bfloat16, device=q.device)   # the caller's output buffer
    rc = fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), bt.data_ptr(), pos.data_ptr(), slot.data_ptr(),
            out.data_ptr(), n, n_q, n_kv, d, page, bt.shape[1], n_pages, window, scale, n_splits,
            torch.cuda.current_stream().cuda_stream)
    return rc, out


def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row():
    from garlic_inference_b200.ops import lib
    fn = _static_entry()
    # two calls in a row on different sizes and slice counts: the second finds the first one's partials
    # in the shared array and must not be disturbed by them
    for seed, lens, n_q, n_kv, d, page, window, splits in [(1, [700, 64, 1, 333, 130], 32, 8, 128, 64, 0, 8),
                                                           (2, [90, 257], 6, 1, 48, 16, 70, 3)]:
        q, k_pool, v_pool, bt, pos, slot = _case(seed, lens, n_q, n_kv, d, page)
        scale = d ** -0.5
        want = K().attention_decode_bf16(q, k_pool, v_pool, bt, pos, slot, scale, window, n_splits=splits)
        rc, got = _call_static(fn, q, k_pool, v_pool, bt, pos, slot, scale, window, splits)
        assert rc == 0, lib().gi_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(got, want), "the same kernels on the same inputs: the same bits"
        # the property the entry point exists for: a further call takes no device memory, from the driver or
        # from torch's allocator (the output buffer is made before the reading)
        n, n_pages = q.shape[0], k_pool.shape[0]
        out = torch.empty((n, n_q * d), dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
        rc = fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), bt.data_ptr(), pos.data_ptr(), slot.data_ptr(),
                out.data_ptr(), n, n_q, n_kv, d, page, bt.shape[1], n_pages, window, scale, splits,
                torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0 and torch.equal(out, want)
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before


def test_static_scratch_entry_refuses_what_does_not_fit():
    from garlic_inference_b200.ops import lib
    fn = _static_entry()
    q, k_pool, v_pool, bt, pos, slot = _case(3, [40] * 40, 32, 8, 128, 64)
    rc, _ = _call_static(fn, q, k_pool, v_pool, bt, pos, slot, 0.1, 0, 32)      # 40 * 32 * 32 * 130 floats > 2 Mi
    assert rc != 0
    msg = lib().gi_last_error().decode()
    assert "fixed array holds 2097152" in msg and "5324800" in msg
    rc, out = _call_static(fn, q, k_pool, v_pool, bt, pos, slot, 0.1, 0, 4)     # and it still works afterwards
    assert rc == 0 and torch.isfinite(out.float()).all()
