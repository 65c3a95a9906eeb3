"""The projection entry point that allocates nothing (``pi_linear_apply_noalloc``).

Who needs it: a caller that runs projections where a device allocation is not
allowed or not affordable - inside a CUDA stream capture (cudaMalloc cannot be
captured), in a loop with a hard latency budget, or in a process that has handed
all device memory to its own pool.  The library's normal projection call grows a
scratch buffer with cudaMalloc when a bigger shape arrives; this variant works
out of a fixed ~3 MiB area that is part of the library image instead.

The test calls it through the C ABI twice in a row - the second call on a
different matrix with fewer activation rows, so anything stale in the shared
scratch area would show - and compares each result with the ordinary entry
point's (same kernels, so the 2e-5 tolerance of the tensor-GEMM tests is generous)
and with the CPU oracle's int8 matmat, so a defect shared by both entry points
would show as well.  Two more cases cover what the entry point exists for: the
very first projection of a fresh context goes through it (its own set-up path),
and a warmed call leaves the amount of free device memory unchanged.
It lives in its own file, collected last, so that a run that stops at the first
failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _device_buffers(torch, M, K, N, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", dtype=torch.float32, generator=g)
    return x, torch.full((M, N), float("nan"), device="cuda"), torch.full((M, N), float("nan"), device="cuda")


def test_noalloc_projection_matches_the_ordinary_one_twice_in_a_row(oracle):
    import torch

    from paged_infer_b200 import api

    ctx = api.Context(0)
    rng = np.random.default_rng(11)
    cases = [(64, 2048, 2560), (17, 5632, 2048)]   # (activation rows, columns, rows): second call is smaller in M
    lins, codes = [], []
    for M, K, N in cases:
        q = rng.integers(-127, 128, (N, K), dtype=np.int8)
        s = (rng.random(N, dtype=np.float32) + 0.5) * 1e-3
        lins.append(api.Projection.int8(ctx, q, s))
        codes.append((q, s))
    for call, ((M, K, N), lin) in enumerate(zip(cases, lins)):
        x, want, got = _device_buffers(torch, M, K, N, 100 + call)
        torch.cuda.synchronize()
        lin.apply_device(x, want, M)            # existing entry point
        lin.apply_device_noalloc(x, got, M)     # the one under test
        ctx.synchronize()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        assert np.isfinite(g).all(), f"call {call}: output not fully written"
        scale = np.maximum(np.abs(w), 1.0)
        assert (np.abs(g - w) / scale).max() < 2e-5, f"call {call}"
        ref = oracle.matmat_i8(x.cpu().numpy(), *codes[call])
        assert (np.abs(g - ref) / np.maximum(np.abs(ref), 1.0)).max() < 2e-5 * max(1.0, (K / 2048.0) ** 0.5), f"call {call} vs the CPU oracle"
    # and once more on the first matrix: the area still holds the second call's planes
    M, K, N = cases[0]
    x, want, got = _device_buffers(torch, M, K, N, 7)
    torch.cuda.synchronize()
    lins[0].apply_device(x, want, M)
    lins[0].apply_device_noalloc(x, got, M)
    ctx.synchronize()
    assert (np.abs(got.cpu().numpy() - want.cpu().numpy()) / np.maximum(np.abs(want.cpu().numpy()), 1.0)).max() < 2e-5
    ctx.close()


def test_noalloc_first_call_on_a_fresh_context_small_batch_and_no_allocation(oracle):
    """The first projection a new context ever runs goes through the allocation-free entry point (so its own set-up,
    not the ordinary call's, prepares the kernels), with 3 activation rows - fewer than the ordinary call would send
    to the tensor path; then a warmed call must leave the free device memory exactly where it was."""
    import torch

    from paged_infer_b200 import api

    torch.cuda.init()
    torch.zeros(1, device="cuda")
    ctx = api.Context(0)
    rng = np.random.default_rng(5)
    M, K, N = 3, 1024, 384
    q = rng.integers(-127, 128, (N, K), dtype=np.int8)
    s = (rng.random(N, dtype=np.float32) + 0.5) * 1e-3
    lin = api.Projection.int8(ctx, q, s)
    x, _, got = _device_buffers(torch, M, K, N, 1)
    torch.cuda.synchronize()
    lin.apply_device_noalloc(x, got, M)          # first projection of this context
    ctx.synchronize()
    ref = oracle.matmat_i8(x.cpu().numpy(), q, s)
    assert (np.abs(got.cpu().numpy() - ref) / np.maximum(np.abs(ref), 1.0)).max() < 2e-5
    x2, _, got2 = _device_buffers(torch, 64, K, N, 2)
    torch.cuda.synchronize()
    lin.apply_device_noalloc(x2, got2, 64)       # warm the widest tile as well
    ctx.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        lin.apply_device_noalloc(x2, got2, 64)
        lin.apply_device_noalloc(x, got, M)
    ctx.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    ctx.close()


def test_noalloc_projection_refuses_what_does_not_fit():
    import torch

    from paged_infer_b200 import api

    ctx = api.Context(0)
    q = np.ones((256, 256), np.int8)
    lin = api.Projection.int8(ctx, q, np.ones(256, np.float32))
    x = torch.zeros(65, 256, device="cuda")
    out = torch.zeros(65, 256, device="cuda")
    with pytest.raises(api.PiError, match="built-in scratch"):
        lin.apply_device_noalloc(x, out, 65)
    wide = api.Projection.int8(ctx, np.ones((128, 8192 + 128), np.int8), np.ones(128, np.float32))
    with pytest.raises(api.PiError, match="built-in scratch"):
        wide.apply_device_noalloc(torch.zeros(4, 8192 + 128, device="cuda"), torch.zeros(4, 128, device="cuda"), 4)
    odd = api.Projection.int8(ctx, np.ones((64, 96), np.int8), np.ones(64, np.float32))
    with pytest.raises(api.PiError, match="multiple of 128"):
        odd.apply_device_noalloc(torch.zeros(4, 96, device="cuda"), torch.zeros(4, 64, device="cuda"), 4)
    lin.apply_device_noalloc(x[:8], out[:8], 8)   # the context is still usable
    ctx.synchronize()
    ctx.close()
