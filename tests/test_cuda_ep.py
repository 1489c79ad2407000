"""Expert-parallel phases on the GPU.  With one GPU the three phase calls in a row must reproduce
uocr_cuda_moe_layer_forward bit for bit (same kernels, exchange elided); with two or more GPUs a torchrun
job checks the sharded layer against the single-GPU layer (tests/ep_two_gpu_check.py)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import quant  # noqa: E402

ROOT = Path(__file__).resolve().parent.parent
FULL = dict(H=1280, E=64, K=6, F=896, S=1792)


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    return entry.load_package()


@pytest.mark.parametrize("qname,n", [("q4_0", 300), ("q8_0", 96)])
def test_phases_on_one_gpu_equal_the_layer_call(pkg, port, qname, n):
    rng = np.random.default_rng(41)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_BY_NAME[qname], logit_bias=quant.zipf_logit_bias(rng, 64), **FULL)
    hidden = quant.synth_activations(rng, n, FULL["H"])
    resid = quant.synth_activations(rng, n, FULL["H"])
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(n)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        d_h = torch.from_numpy(hidden).cuda().view(torch.float16)
        d_r = torch.from_numpy(resid).cuda().view(torch.float16)
        want = torch.zeros_like(d_h)
        ids = torch.zeros((n, 6), dtype=torch.int32, device="cuda")
        ctx.layer_forward(0, d_h, n, want, residual=d_r, top_ids=ids)
        ctx.synchronize()
        layer = pkg.ep.ExpertParallelLayer(ctx, 0, 64, 6, FULL["H"])
        out = torch.zeros_like(d_h)
        plan = layer.forward(d_h, out, residual=d_r)
        ctx.synchronize()
        assert torch.equal(out, want)
        # the per-expert counts the dispatch phase reports are the histogram of the routing
        hist = np.bincount(ids.cpu().numpy().reshape(-1), minlength=64)
        assert np.array_equal(plan.send_counts.reshape(-1), hist) and plan.rows_received == n * 6
        assert ctx.kernel_launches > 0
    # and the layer itself matches the oracle (routing on GPU logits: compare rows routed identically)
    o = port.layer(L, hidden, resid, threads=16)
    same = np.all(ids.cpu().numpy().view(np.uint32) == o.ids, axis=1)
    got = out.cpu().numpy().astype(np.float32)
    assert same.mean() > 0.97
    assert np.max(np.abs(got[same] - o.out[same])) <= 2e-2


def test_peer_memory_phases_on_one_gpu_equal_the_layer_call(pkg):
    """The peer-memory form of the phases with a group of one rank: the scatter writes into this rank's own exchange
    buffer and the combine reads from it; the result equals uocr_cuda_moe_layer_forward bit for bit, twice in a row."""
    rng = np.random.default_rng(43)
    n = 300
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q4_0, logit_bias=quant.zipf_logit_bias(rng, 64), **FULL)
    hidden = quant.synth_activations(rng, n, FULL["H"])
    resid = quant.synth_activations(rng, n, FULL["H"])
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(n)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        d_h = torch.from_numpy(hidden).cuda().view(torch.float16)
        d_r = torch.from_numpy(resid).cuda().view(torch.float16)
        want = torch.zeros_like(d_h)
        ctx.layer_forward(0, d_h, n, want, residual=d_r)
        layer = pkg.ep.PeerExpertParallelLayer(ctx, 0, FULL["E"], FULL["K"], FULL["H"], row_capacity=n * FULL["K"])
        for call in (layer.forward, layer.forward_collectives, layer.forward_host_counts, layer.forward):   # ranks synchronised on the device / by collectives / offsets on the host
            got = torch.zeros_like(d_h)
            call(d_h, got, residual=d_r)
            ctx.synchronize()
            assert layer.last_plan.rows_received == n * FULL["K"]
            assert torch.equal(got, want)
        # offsets that point outside the buffer are refused on the device, not dereferenced
        ctx.ep_peer_dispatch(0, d_h, n, layer._offsets)
        ctx.ep_peer_scatter(0, d_h, n, np.full(64, n * FULL["K"], np.uint32))
        with pytest.raises(pkg.UocrCudaError, match="exchange buffers"):
            ctx.synchronize()
        layer.close()


def test_experts_phase_rejects_more_rows_than_the_arena_holds(pkg):
    rng = np.random.default_rng(42)
    L = quant.synth_layer(rng, expert_qtype=quant.QTYPE_Q8_0, **FULL)
    with pkg.Context() as ctx:
        ctx.map_layer(L)
        ctx.allocate_runtime_arenas(16)
        rows = torch.zeros((16, FULL["H"]), dtype=torch.float16, device="cuda")
        counts = np.zeros((2, 32), np.uint32)
        counts[1, 3] = 16 * 6 + 1
        with pytest.raises(pkg.UocrCudaError, match="exceed the arena capacity"):
            ctx.ep_experts(0, 32, 32, counts, rows, rows)
        with pytest.raises(pkg.UocrCudaError, match="invalid expert range"):
            ctx.ep_experts(0, 48, 32, counts, rows, rows)


def test_two_gpu_expert_parallel_equals_single_gpu(pkg):
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs two GPUs")
    world = 2
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + os.getpid() % 1000), str(ROOT / "tests" / "ep_two_gpu_check.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("EP_OK") == world, res.stdout[-3000:]
