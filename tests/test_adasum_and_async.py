"""Adasum closed forms and numerical stability, and asynchronous fused
allreduce with poll() (parity: test/parallel/test_adasum_pytorch.py:47-211,
test/parallel/test_torch.py:251-295)."""
import torch

from parallel_utils import run_parallel


def _adasum_closed_forms(rank, size):
    import horovod_b200.torch as hvd
    hvd.init()
    res = {}
    n = 64
    # orthogonal inputs: Adasum is the plain sum
    x = torch.zeros(n, dtype=torch.float64)
    x[rank * 8:(rank + 1) * 8] = rank + 1.0
    out = hvd.allreduce(x, op=hvd.Adasum, name="orth")
    exp = torch.zeros(n, dtype=torch.float64)
    for r in range(size):
        exp[r * 8:(r + 1) * 8] = r + 1.0
    res["orthogonal_is_sum"] = torch.allclose(out, exp, atol=1e-12)
    # identical (parallel) inputs: Adasum is the average = the input itself
    y = torch.linspace(-1, 1, n, dtype=torch.float64)
    res["parallel_is_average"] = torch.allclose(hvd.allreduce(y.clone(), op=hvd.Adasum,
                                                              name="par"), y, atol=1e-12)
    # anti-parallel inputs of equal norm: a + b = 0 and each coefficient is 1.5 -> 0
    z = y if rank % 2 == 0 else -y
    res["antiparallel"] = hvd.allreduce(z.clone(), op=hvd.Adasum, name="anti").abs().max() < 1e-12
    # zero vectors do not divide by zero
    res["zeros"] = bool((hvd.allreduce(torch.zeros(n), op=hvd.Adasum, name="zero") == 0).all())
    # one rank zero, the other not: the result is the non-zero one
    w = torch.ones(n, dtype=torch.float64) * (1.0 if rank == 0 else 0.0)
    res["one_zero"] = torch.allclose(hvd.allreduce(w, op=hvd.Adasum, name="onezero"),
                                     torch.ones(n, dtype=torch.float64), atol=1e-12)
    # tiny and huge magnitudes stay finite and scale-equivariant
    base = torch.randn(n, generator=torch.Generator().manual_seed(3 + rank), dtype=torch.float64)
    ref = hvd.allreduce(base.clone(), op=hvd.Adasum, name="scale.ref")
    for tag, s in (("tiny", 1e-60), ("huge", 1e150)):
        got = hvd.allreduce(base * s, op=hvd.Adasum, name="scale.%s" % tag)
        res[tag] = bool(torch.isfinite(got).all()) and torch.allclose(got / s, ref, rtol=1e-9,
                                                                       atol=1e-12)
    # below sqrt(DBL_MIN) a squared norm counts as zero and the vectors are just
    # added (horovod/common/ops/adasum/adasum.h:380-397)
    got = hvd.allreduce(base * 1e-160, op=hvd.Adasum, name="scale.underflow")
    both = sum(torch.randn(n, generator=torch.Generator().manual_seed(3 + r),
                           dtype=torch.float64) for r in range(size)) * 1e-160
    res["underflow_adds"] = torch.allclose(got, both, rtol=1e-9, atol=0)
    # fp16 storage: computed in wider precision, finite for values near the fp16 range
    h = (torch.ones(n) * 200.0).half()
    got = hvd.allreduce(h, op=hvd.Adasum, name="half")
    res["fp16"] = got.dtype == torch.float16 and bool(torch.isfinite(got.float()).all()) \
        and abs(float(got[0]) - 200.0) < 1.0
    # several tensors in one fused response keep their own coefficients
    a = hvd.allreduce_async(x.clone(), op=hvd.Adasum, name="fuse.orth")
    b = hvd.allreduce_async(y.clone(), op=hvd.Adasum, name="fuse.par")
    res["fused_independent"] = torch.allclose(hvd.synchronize(a), exp, atol=1e-12) and \
        torch.allclose(hvd.synchronize(b), y, atol=1e-12)
    hvd.shutdown()
    return res


def test_adasum_closed_forms_and_stability():
    for rep in run_parallel(_adasum_closed_forms, np=2, timeout=300):
        bad = [k for k, v in rep.items() if not v]
        assert not bad, bad


def _adasum_in_small_pieces(rank, size):
    import os
    # 100-byte pieces: every exchange of halves takes several, of uneven length
    os.environ["HOROVOD_ADASUM_MPI_CHUNK_SIZE"] = "100"
    import horovod_b200.torch as hvd
    hvd.init()
    n = 1000 + 7
    mine = torch.randn(n, generator=torch.Generator().manual_seed(40 + rank), dtype=torch.float64)
    got = hvd.allreduce(mine.clone(), op=hvd.Adasum, name="pieces")
    vectors = [torch.randn(n, generator=torch.Generator().manual_seed(40 + r), dtype=torch.float64)
               for r in range(size)]
    while len(vectors) > 1:  # the same pairwise tree on whole vectors
        nxt = []
        for a, b in zip(vectors[0::2], vectors[1::2]):
            dot, na, nb = float(a @ b), float(a @ a), float(b @ b)
            nxt.append((1 - dot / (2 * na)) * a + (1 - dot / (2 * nb)) * b)
        vectors = nxt
    hvd.shutdown()
    return bool(torch.allclose(got, vectors[0], rtol=1e-10, atol=1e-12))


def test_adasum_exchanges_in_pieces_of_the_chunk_size():
    assert all(run_parallel(_adasum_in_small_pieces, np=4, timeout=300))


def _async_fused(rank, size):
    import time
    import horovod_b200.torch as hvd
    hvd.init()
    ok, saw_pending = True, False
    for dtype in (torch.int32, torch.float32, torch.float64):
        handles, expected = [], []
        for i in range(40):
            t = (torch.arange(1000 + i) % 17).to(dtype) * (rank + 1)
            handles.append(hvd.allreduce_async(t, op=hvd.Sum, name="af.%s.%d" % (dtype, i)))
            expected.append((torch.arange(1000 + i) % 17).to(dtype) * sum(range(1, size + 1)))
        for h in handles:
            if not hvd.poll(h):
                saw_pending = True
                while not hvd.poll(h):
                    time.sleep(0.0005)
        for h, e in zip(handles, expected):
            ok = ok and torch.equal(hvd.synchronize(h), e)
    hvd.shutdown()
    return ok, saw_pending


def test_async_fused_allreduce_with_poll():
    out = run_parallel(_async_fused, np=2, timeout=300)
    assert all(o[0] for o in out)
    # the ops are asynchronous: at least one handle was still in flight when polled
    assert any(o[1] for o in out)
