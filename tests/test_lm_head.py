"""The LM head fused with its argmax (uocr_cuda_lm_head_argmax) against the CPU oracle: the token id of the largest
logit per token, ties to the lowest id, NaN rows skipped.  Integer result: compared exactly, except where the two
largest CPU logits lie closer than the rounding of a 1280-term f32 sum (the GPU sums in another order), in which case
either of the two ids is accepted; scores within 1e-4 relative."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

from oracle import quant  # noqa: E402

VOCAB, H = 129280, 1280      # UOCR_VOCAB_SIZE, UOCR_HIDDEN_SIZE (src/model/uocr_constants.h:6, :21)


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; the library has no CPU path")
    torch.cuda.set_device(0)
    return entry.load_package()


@pytest.fixture(scope="module")
def full_weights():
    rng = np.random.default_rng(500)
    return rng.standard_normal((VOCAB, H), dtype=np.float32) * 0.02


def run(pkg, m, x_bits):
    n = x_bits.shape[0]
    with pkg.Context() as ctx:
        ctx.map_lm_head(m)
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)
        ids = torch.full((n,), 7, dtype=torch.int32, device="cuda")
        scores = torch.zeros((n,), dtype=torch.float32, device="cuda")
        d_x = torch.from_numpy(x_bits).cuda().view(torch.float16)
        for _ in range(2):                       # twice: the ticket of the first call must be back at zero
            ctx.lm_head_argmax(d_x, n, ids, scores)
        ctx.synchronize()
        return ids.cpu().numpy().view(np.uint32), scores.cpu().numpy()


@pytest.mark.parametrize("qname", ["q4_0", "q8_0"])
@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_full_vocabulary_argmax(pkg, port, full_weights, qname, n):
    m = quant.make_matrix(quant.QTYPE_BY_NAME[qname], full_weights)
    x = quant.synth_activations(np.random.default_rng(510 + n), n, H)
    got_ids, got_scores = run(pkg, m, x)
    want_ids, want_scores, logits = port.lm_head_argmax(m, x, want_logits=True)
    for t in range(n):
        if got_ids[t] != want_ids[t]:            # only acceptable when the CPU itself sees a near-tie
            top2 = np.sort(logits[t])[-2:]
            assert abs(top2[1] - top2[0]) <= 2e-5 * max(1.0, abs(top2[1])), (t, got_ids[t], want_ids[t], top2)
            assert abs(logits[t, got_ids[t]] - top2[1]) <= 2e-5 * max(1.0, abs(top2[1]))
        assert abs(got_scores[t] - logits[t, got_ids[t]]) <= 1e-4 * max(1.0, abs(want_scores[t]))


@pytest.mark.parametrize("qname", ["q4_0", "q8_0"])
@pytest.mark.parametrize("V,Hc", [(1000, 1280), (4096, 1280), (64, 256), (2384, 2048)])
def test_other_shapes(pkg, port, qname, V, Hc):
    """1000 rows (not a multiple of 16) go through the row-per-lane-group kernel, the others through the bulk-copy ring:
    with fewer 16-row blocks than CTAs (64 rows), one or two blocks per CTA, and the widest hidden size."""
    rng = np.random.default_rng(540 + V)
    m = quant.make_matrix(quant.QTYPE_BY_NAME[qname], rng.standard_normal((V, Hc), dtype=np.float32) * 0.05)
    x = quant.synth_activations(rng, 3, Hc)
    got_ids, got_scores = run(pkg, m, x)
    want_ids, want_scores, logits = port.lm_head_argmax(m, x, want_logits=True)
    for t in range(3):
        if got_ids[t] != want_ids[t]:
            top2 = np.sort(logits[t])[-2:]
            assert abs(top2[1] - top2[0]) <= 2e-5 * max(1.0, abs(top2[1])), (t, got_ids[t], want_ids[t], top2)
        assert abs(got_scores[t] - logits[t, got_ids[t]]) <= 1e-4 * max(1.0, abs(want_scores[t]))


def test_ties_go_to_the_lowest_id_and_nan_rows_are_skipped(pkg, port):
    rng = np.random.default_rng(520)
    w = rng.standard_normal((4096, H), dtype=np.float32) * 0.02
    x = quant.synth_activations(rng, 2, H)
    m0 = quant.make_matrix(quant.QTYPE_F16, w)
    ids0, _, logits = port.lm_head_argmax(m0, x, want_logits=True)
    best = int(ids0[0])
    twin = (best + 1000) % 4096                            # an exact copy of token 0's best row at another index
    w2 = w.copy()
    w2[twin] = w2[best]
    m = quant.make_matrix(quant.QTYPE_F16, w2)
    got, _ = run(pkg, m, x)
    want, _, _ = port.lm_head_argmax(m, x)
    assert np.array_equal(got, want)
    assert got[0] == min(best, twin)
    # a row with a NaN weight has a NaN logit and never wins, wherever it is
    bits = m.qweight.view(np.uint16).reshape(4096, H).copy()
    bits[int(want[1]), 5] = 0x7E00
    m_nan = quant.Matrix(quant.QTYPE_F16, 4096, H, bits.view(np.uint8).reshape(-1), None)
    got_nan, _ = run(pkg, m_nan, x)
    want_nan, _, _ = port.lm_head_argmax(m_nan, x)
    assert np.array_equal(got_nan, want_nan) and got_nan[1] != want[1]


def test_lm_head_argument_checks(pkg):
    rng = np.random.default_rng(530)
    m = quant.make_matrix(quant.QTYPE_Q8_0, rng.standard_normal((256, 128), dtype=np.float32))
    with pkg.Context() as ctx:
        ids = torch.zeros(8, dtype=torch.int32, device="cuda")
        x = torch.zeros((8, 128), dtype=torch.float16, device="cuda")
        with pytest.raises(pkg.UocrCudaError, match="no LM head"):
            ctx.lm_head_argmax(x, 1, ids)
        ctx.map_lm_head(m)
        with pytest.raises(pkg.UocrCudaError, match="already mapped"):
            ctx.map_lm_head(m)
        with pytest.raises(pkg.UocrCudaError, match="at most 4"):
            ctx.lm_head_argmax(x, 5, ids)
        ctx.lm_head_argmax(x, 4, ids)            # all-zero activations: every logit is 0, the lowest id wins
        ctx.synchronize()
        assert ids[:4].tolist() == [0, 0, 0, 0]
        ctx.unmap_model()
        with pytest.raises(pkg.UocrCudaError, match="no LM head"):
            ctx.lm_head_argmax(x, 1, ids)
