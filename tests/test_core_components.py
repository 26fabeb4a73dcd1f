"""Unit tests of the native core's building blocks through `_C.testing`:
software float conversions against torch, wire format, CPU reduction kernels,
response cache / coordinator, stall inspector, Gaussian process, Bayesian
optimisation and the autotuning parameter manager."""
import math
import struct

import numpy as np
import pytest
import torch

from horovod_b200 import _C

T = _C.testing
U8, I8, U16, I16, I32, I64, F16, F32, F64, BOOL, BF16 = range(11)
AVG, SUM, ADASUM, MIN, MAX, PROD = range(6)


def test_half_and_bf16_conversions_match_torch():
    g = torch.Generator().manual_seed(0)
    vals = torch.cat([torch.randn(2000, generator=g) * 10 ** torch.randint(-8, 6, (2000,), generator=g).float(),
                      torch.tensor([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 5.96e-8, 2.98e-8,
                                    float("inf"), -float("inf"), 1.0, 0.1, 3.14159])])
    for v in vals.tolist():
        bits = T.float_to_half_bits(v)
        want = torch.tensor(v).half().view(torch.int16).item() & 0xFFFF
        assert bits == want, (v, bits, want)
        bb = T.float_to_bf16_bits(v)
        wantb = torch.tensor(v).bfloat16().view(torch.int16).item() & 0xFFFF
        assert bb == wantb, (v, bb, wantb)
    for bits in list(range(0, 0x7C00, 37)) + [0x8001, 0xFBFF, 0x0001, 0x03FF, 0x0400]:
        want = torch.tensor([bits], dtype=torch.uint16).view(torch.float16).float().item()
        assert T.half_bits_to_float(bits) == want
    assert math.isnan(T.half_bits_to_float(T.float_to_half_bits(float("nan"))))
    assert T.bf16_bits_to_float(0x3F80) == 1.0


def test_wire_roundtrip_and_garbage():
    out = T.wire_roundtrip("layer.weight", [3, 4, 5], BF16, 0.5, 0.125)
    (name, shape, dtype, pre, post, rank, rtype, root, device, group, op, shutdown,
     names, err, sizes, joined, ptype, nbytes) = out
    assert (name, shape, dtype, pre, post) == ("layer.weight", [3, 4, 5], BF16, 0.5, 0.125)
    assert (rank, rtype, root, device, group, op, shutdown) == (3, 1, 2, 1, 7, MAX, True)
    assert names == ["layer.weight", "layer.weight2"] and err == "boom"
    assert sizes == [5, 6, 7] and joined == 4 and ptype == 7
    assert not T.wire_parse_garbage(b"\x00\x05\x00\x00\x00garbage")
    assert not T.wire_parse_garbage(b"")


def test_cpu_reduce_and_scale_kernels():
    rng = np.random.default_rng(0)
    for dtype, npdt in [(F32, np.float32), (F64, np.float64), (I32, np.int32), (I64, np.int64),
                        (U8, np.uint8), (I16, np.int16)]:
        a = rng.integers(1, 9, 37).astype(npdt)
        b = rng.integers(1, 9, 37).astype(npdt)
        for op, fn in [(SUM, np.add), (MIN, np.minimum), (MAX, np.maximum), (PROD, np.multiply)]:
            got = np.frombuffer(T.reduce_into(a.tobytes(), b.tobytes(), 37, dtype, op), npdt)
            assert np.array_equal(got, fn(a, b).astype(npdt)), (dtype, op)
    a = torch.randn(1001).half()
    b = torch.randn(1001).half()
    got = torch.frombuffer(bytearray(T.reduce_into(a.numpy().tobytes(), b.numpy().tobytes(),
                                                    1001, F16, SUM)), dtype=torch.float16)
    assert torch.equal(got, (a.float() + b.float()).half())
    a = torch.randn(1001).bfloat16()
    b = torch.randn(1001).bfloat16()
    got = torch.frombuffer(bytearray(T.reduce_into(a.view(torch.int16).numpy().tobytes(),
                                                    b.view(torch.int16).numpy().tobytes(),
                                                    1001, BF16, SUM)), dtype=torch.bfloat16)
    assert torch.equal(got, (a.float() + b.float()).bfloat16())
    x = np.arange(10, dtype=np.float32)
    assert np.allclose(np.frombuffer(T.scale_buffer(x.tobytes(), 10, F32, 0.25), np.float32), x / 4)
    xi = np.arange(10, dtype=np.int32)
    assert np.array_equal(np.frombuffer(T.scale_buffer(xi.tobytes(), 10, I32, 0.5), np.int32), xi // 2)


def test_adasum_pair_closed_forms():
    a = [1.0, 0.0, 0.0, 2.0]
    b = [0.0, 3.0, 0.0, 0.0]
    # orthogonal -> sum
    assert T.adasum_pair(a, [0.0, 3.0, 4.0, 0.0]) == [1.0, 3.0, 4.0, 2.0]
    # identical -> the same vector (average of equals)
    assert np.allclose(T.adasum_pair(a, a), a)
    # zero vector leaves the other untouched
    assert T.adasum_pair(a, [0.0] * 4) == a
    assert np.allclose(T.adasum_pair(b, [0.0, 6.0, 0.0, 0.0]), [0.0, 4.5, 0.0, 0.0])


def test_response_cache_hit_invalid_lru():
    h = T.CacheHarness()
    h.set_capacity(3)
    MISS, HIT, INVALID = 0, 1, 2
    assert h.cached("a", [4], F32) == MISS
    for n in "abc":
        h.put(n, [4], F32)
    assert h.num_bits() == 3
    assert h.cached("a", [4], F32) == HIT
    assert h.cached("a", [5], F32) == INVALID
    assert h.cached("a", [4], F16) == INVALID
    # "a" is the least recently used: inserting "d" evicts it
    h.put("d", [4], F32)
    assert not h.has("a") and h.has("d") and h.num_bits() == 3
    # touching "b" protects it from the next eviction
    h.touch(h.bit("b"))
    h.put("e", [4], F32)
    assert h.has("b") and not h.has("c")
    # bits stay a dense range
    assert sorted(h.bit(n) for n in "bde") == [0, 1, 2]
    h.erase(h.bit("d"))
    assert sorted(h.bit(n) for n in "be") == [0, 1]


def test_cache_coordinator_sync_semantics():
    out = T.coordinate(70, [([0, 5, 69], [], False, False),
                            ([0, 69], [], False, True),
                            ([0, 5, 69, 7], [], False, False)])
    for hits, invalid, shutdown, uncached in out:
        assert hits == [0, 69] and invalid == [] and not shutdown and uncached
    out = T.coordinate(8, [([1, 2], [2], False, False), ([1, 2], [], True, False)])
    for hits, invalid, shutdown, uncached in out:
        assert hits == [1] and invalid == [2] and shutdown


def test_stall_inspector_names_missing_ranks():
    s = T.StallHarness()
    s.configure(0, 0)
    s.record("grad.7", 0, 4)
    s.record("grad.7", 2, 4)
    import time
    time.sleep(1.1)
    shutdown, report = s.check([10, 11, 12, 13])
    assert not shutdown
    assert "grad.7" in report and "[11, 13]" in report
    s.configure(0, 1)
    time.sleep(1.0)
    shutdown, _ = s.check([10, 11, 12, 13])
    assert shutdown
    s.remove("grad.7")
    shutdown, _ = s.check([10, 11, 12, 13])
    assert not shutdown


def test_gaussian_process_interpolates():
    gp = T.GaussianProcess(1e-6)
    xs = [[x / 10.0] for x in range(11)]
    ys = [math.sin(3 * x[0]) for x in xs]
    gp.fit(xs, ys)
    for x in [0.05, 0.33, 0.71]:
        mean, sd = gp.predict([x])
        assert abs(mean - math.sin(3 * x)) < 0.02 and sd < 0.1
    _, sd_far = gp.predict([3.0])
    assert sd_far > 0.5


def test_bayesian_optimization_finds_the_peak():
    def f(x, y):
        return -((x - 30) ** 2) / 400 - ((y - 12) ** 2) / 100

    bo = T.BayesianOptimization([(0.0, 64.0), (1.0, 100.0)], alpha=1e-4, seed=1)
    for x, y in [(4, 5), (32, 50), (16, 25), (8, 10)]:
        bo.add_sample([float(x), float(y)], f(x, y))
    for _ in range(25):
        x, y = bo.next_sample()
        assert 0 <= x <= 64 and 1 <= y <= 100
        bo.add_sample([x, y], f(x, y))
    bx, by = bo.best_x()
    assert abs(bx - 30) < 8 and abs(by - 12) < 8, (bx, by)


def test_parameter_manager_tunes_and_stops(tmp_path):
    log = tmp_path / "autotune.csv"
    pm = T.ParameterManager()
    pm.set_warmup_samples(0)
    pm.set_steps_per_sample(1)
    pm.set_bayes_opt_max_samples(4)
    pm.set_hierarchical_allreduce(False, True)
    pm.set_hierarchical_allgather(False, True)
    pm.initialize(0, 0, str(log))
    pm.set_auto_tuning(True)
    changes = 0
    seen = set()
    for step in range(2000):
        if not pm.is_auto_tuning():
            break
        if pm.update(["t0", "t1"], 1 << 20):
            changes += 1
            seen.add((pm.fusion_threshold(), round(pm.cycle_time_ms(), 3), pm.cache_enabled()))
    assert not pm.is_auto_tuning(), "tuning should finish"
    assert changes >= 5 and len(seen) >= 4
    assert 0 <= pm.fusion_threshold() <= 256 << 20 and 1.0 <= pm.cycle_time_ms() <= 100.0
    rows = log.read_text().strip().splitlines()
    assert rows[0].startswith("hierarchical_allreduce") and len(rows) >= 6
    # an explicitly fixed knob is never touched
    pm2 = T.ParameterManager()
    pm2.set_warmup_samples(0)
    pm2.set_steps_per_sample(1)
    pm2.set_bayes_opt_max_samples(3)
    pm2.set_fusion_threshold(12345678, True)
    pm2.set_cache_enabled(True, True)
    pm2.set_hierarchical_allreduce(False, True)
    pm2.set_hierarchical_allgather(False, True)
    pm2.initialize(0, 0, "")
    pm2.set_auto_tuning(True)
    for step in range(500):
        pm2.update(["t0"], 1000)
        assert pm2.fusion_threshold() == 12345678 and pm2.cache_enabled()


def test_fusion_policy_threshold_lookahead_and_compatibility():
    """Parity: FuseResponses, horovod/common/controller.cc:793-930."""
    AR, BC, F32, F16 = 0, 2, 7, 6  # Response types / dtype ids of the wire format

    def item(name, n, dtype=F32, pre=1.0, post=1.0, typ=AR, root=0):
        return (typ, name, n, dtype, pre, post, root)

    # everything fits: one fused response, order kept
    assert T.fuse_responses([item("a", 10), item("b", 20), item("c", 30)], 1 << 20) == \
        [["a", "b", "c"]]
    # 16-byte rounding: 3 tensors of 5 floats = 3 x 32 bytes; threshold 64 holds two
    assert T.fuse_responses([item("a", 5), item("b", 5), item("c", 5)], 64) == [["a", "b"], ["c"]]
    # look-ahead: an fp16 response between two fp32 ones is skipped, not a barrier,
    # and keeps its place in the queue
    assert T.fuse_responses([item("w1", 100), item("h", 100, F16), item("w2", 100)], 1 << 20) == \
        [["w1", "w2"], ["h"]]
    # look-ahead stops when the skipped bytes would not have fitted either
    assert T.fuse_responses([item("w1", 100), item("big", 1000, F16), item("w2", 100)], 1024) == \
        [["w1"], ["big"], ["w2"]]
    # different scale factors do not fuse
    assert T.fuse_responses([item("a", 10), item("b", 10, post=0.5), item("c", 10)], 1 << 20) == \
        [["a", "c"], ["b"]]
    # a tensor larger than the threshold travels alone
    assert T.fuse_responses([item("huge", 1 << 20), item("s", 4)], 1024) == [["huge"], ["s"]]
    # broadcasts fuse per root, whatever the dtype
    assert T.fuse_responses([item("p", 8, F32, typ=BC, root=0), item("q", 8, F16, typ=BC, root=0),
                             item("r", 8, F32, typ=BC, root=1)], 1 << 20) == [["p", "q"], ["r"]]
    # threshold 0: nothing fuses
    assert T.fuse_responses([item("a", 1), item("b", 1)], 0) == [["a"], ["b"]]
    # reduce-scatters fuse among themselves under the rules of a reduction
    # (dtype and scaling must agree), never with an allreduce; alltoalls never fuse
    RS, A2A = 6, 5
    assert T.fuse_responses([item("r1", 10, typ=RS), item("x", 10), item("r2", 10, typ=RS),
                             item("r3", 10, typ=RS, post=0.5), item("r4", 10, F16, typ=RS)],
                            1 << 20) == [["r1", "r2"], ["x"], ["r3"], ["r4"]]
    assert T.fuse_responses([item("t1", 10, typ=A2A), item("t2", 10, typ=A2A)], 1 << 20) == \
        [["t1"], ["t2"]]


def test_build_and_extension_queries(monkeypatch):
    """Parity: horovod/common/util.py:33-211 (extension path and check, build
    feature queries, env context manager)."""
    import os
    import horovod_b200
    from horovod_b200.common import util
    path = util.get_extension_full_path(horovod_b200.__file__, "_C")
    assert os.path.exists(path) and path.endswith(".so")
    util.check_extension("horovod_b200.torch", "HOROVOD_WITH_PYTORCH", horovod_b200.__file__, "_C")
    with pytest.raises(ImportError, match="build_ext"):
        util.check_extension("horovod_b200.nope", "HOROVOD_WITH_NOPE", horovod_b200.__file__, "_nope")
    assert util.extension_available() and util.gloo_built() and util.nccl_built()
    assert not util.mpi_built() and not util.ddl_built() and not util.ccl_built()
    monkeypatch.delenv("HVD_UTIL_PROBE", raising=False)
    with util.env(HVD_UTIL_PROBE=3):
        assert os.environ["HVD_UTIL_PROBE"] == "3"
    assert "HVD_UTIL_PROBE" not in os.environ
    import horovod_b200.torch as hvd
    assert hvd.check_extension is util.check_extension


def test_thread_affinity_value_is_one_core_or_one_per_local_rank():
    t = _C.testing
    assert t.affinity_core("", 0) == -1
    assert t.affinity_core("5", 0) == 5 and t.affinity_core("5", 3) == 5
    assert [t.affinity_core("0,2,4,6", r) for r in range(4)] == [0, 2, 4, 6]
    assert t.affinity_core("0,2", 2) == -1          # no entry for this local rank
    assert t.affinity_core("0,x", 1) == -1 and t.affinity_core("-3", 0) == -1


def test_elastic_wait_polls_nccl_for_asynchronous_errors_and_aborts():
    """The host-side wait of an elastic job for a device collective, with a
    stand-in for NCCL's error reporting (no GPU, no fault): without an error
    it ends when the work is done and touches nothing; when a communicator
    reports an error, all are aborted once, the wait ends with that error
    after the aborted work has drained (or after the grace period), and the
    set stays marked failed until it is destroyed."""
    t = _C.testing
    ok, msg, polls, queries, aborted, empty, failed, destroyed, failed_after = \
        t.nccl_async_wait(3, -1, 0, 5, 0)
    assert (ok, msg, polls, aborted, empty, failed) == (True, "", 5, 0, False, False)
    assert destroyed == 3 and not failed_after
    # communicator 1 fails at its 4th query: 4 polls without completion, then the abort
    ok, msg, polls, queries, aborted, empty, failed, destroyed, failed_after = \
        t.nccl_async_wait(3, 1, 4, 10 ** 9, 3)
    assert not ok and "asynchronous error" in msg and "peer is gone (fake)" in msg
    assert queries == 4 and aborted == 3 and empty and failed
    assert polls == 4 + 3          # three more polls until the aborted work has drained
    assert destroyed == 0 and not failed_after   # nothing left to destroy; the mark is cleared
    # the work never drains: the wait still ends, after the grace period, with the error
    ok, msg, polls, *_ = t.nccl_async_wait(1, 0, 1, 10 ** 9, 10 ** 9)
    assert not ok and "aborted" in msg and polls > 3


def test_response_path_counters_are_readable_without_a_gpu():
    import horovod_b200.utils as utils
    paths = utils.response_paths()
    assert set(paths) == {"symm", "nccl"} and all(isinstance(v, int) and v >= 0
                                                  for v in paths.values())
