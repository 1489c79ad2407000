"""The allocation-free dispatch plan (uocr_cuda_moe_dispatch_plan_noalloc).

Some hosts of the library cannot call cudaMalloc at the point where they need the token-to-expert
permutation: they sit on a hot path guarded against allocation, run a decode loop with a frozen memory map, or their
engine has already given away the whole device budget.  This entry point needs no context and no arena;
its scratch is a fixed array inside the library.  The test calls it through the C ABI twice in a row on
different inputs and compares every output with the regular entry point's (integer data: exact match),
then checks that sizes beyond its stated limits are refused with a message.

This file is collected last on purpose: a failure here cannot hide the other tests from a run that
stops at the first failure.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import quant  # noqa: E402


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    return entry.load_package()


def random_ids(rng, n, K, E):
    ids = np.stack([rng.permutation(E)[:K] for _ in range(n)]).astype(np.uint32)
    if n > 8:
        ids[3, 0] = 0xFFFFFFFF      # dropped pairs behave the same in both entry points
        ids[6, K - 1] = E
    return ids


def plan_buffers(n, K, E):
    return (torch.full((E + 1,), -1, dtype=torch.int32, device="cuda"),
            torch.full((n * K,), -1, dtype=torch.int32, device="cuda"),
            torch.full((n * K,), -7, dtype=torch.int32, device="cuda"))


def test_noalloc_plan_equals_regular_plan_twice_in_a_row(pkg):
    rng = np.random.default_rng(2024)
    stream = torch.cuda.current_stream().cuda_stream
    # the regular entry point needs a context with a mapped layer and an arena
    L = quant.synth_layer(rng, H=128, E=64, K=6, F=64, S=64, expert_qtype=quant.QTYPE_F16)
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(4096)
        ctx.set_stream(stream)
        for n, K, E in ((300, 6, 64), (4096, 6, 64)):       # two calls in a row, the second larger: stale
            ids = random_ids(rng, n, K, E)                  # scratch contents must not matter
            d_ids = torch.from_numpy(ids.view(np.int32)).cuda()
            want = plan_buffers(n, K, E)
            ctx.dispatch_plan(d_ids, n, K, E, *want)
            ctx.synchronize()
            got = plan_buffers(n, K, E)
            # free device memory as the driver reports it (cudaMemGetInfo): it would also move if the library itself
            # called cudaMalloc, which torch's own allocator statistics cannot see
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            pkg.ffi.dispatch_plan_noalloc(d_ids, n, K, E, *got, cuda_stream=stream)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before
            kept = int(want[0][E].item())
            assert torch.equal(got[0], want[0])                               # expert offsets
            assert torch.equal(got[1][:kept], want[1][:kept])                 # pairs grouped by expert
            assert torch.equal(got[2], want[2])                               # inverse map
            off, rows, inv = quant.stable_dispatch_plan(ids, E)               # and both equal the stable sort
            assert np.array_equal(got[0].cpu().numpy().view(np.uint32), off)
            assert np.array_equal(got[1].cpu().numpy().view(np.uint32)[:kept], rows)
            assert np.array_equal(got[2].cpu().numpy().view(np.uint32), inv)


def test_noalloc_plan_refuses_sizes_beyond_its_scratch(pkg):
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.UocrCudaError, match="256 experts"):
        pkg.ffi.dispatch_plan_noalloc(dummy, 1, 1, 257, dummy, dummy, dummy)
    with pytest.raises(pkg.UocrCudaError, match="1048576 pairs"):
        pkg.ffi.dispatch_plan_noalloc(dummy, 1 << 20, 2, 64, dummy, dummy, dummy)
    with pytest.raises(pkg.UocrCudaError, match="null"):
        pkg.ffi.dispatch_plan_noalloc(None, 1, 1, 8, dummy, dummy, dummy)
    with pytest.raises(pkg.UocrCudaError, match="invalid"):
        pkg.ffi.dispatch_plan_noalloc(dummy, 1, 9, 8, dummy, dummy, dummy)
