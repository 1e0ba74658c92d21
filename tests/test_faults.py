"""Failure detection and recovery, injected on the host only (no GPU is faulted, trapped or hung).

Failures made here: a compressor that raises, a request cancelled mid-flight, an aborted step,
a step that overruns its deadline, a rank that stops beating, a rank that leaves, and a
collective whose peer never joins (gloo ranks with a short process-group timeout).
"""
import multiprocessing as mp
import os
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist

from fastcache_b200 import LLM, SamplingParams
from fastcache_b200.compress import KVCacheLinearDecoupleCompressor
from fastcache_b200.engine.sequence import CompressionState
from fastcache_b200.utils.watchdog import (DeviceWaitTimeout, RankFailure, RankHeartbeat, StepDeadlineExceeded,
                                           StepWatchdog)
from helpers import random_compressor, tiny_llama_config


def _prompts(n=4, length=96, vocab=1024, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, vocab, (length,), generator=g).tolist() for _ in range(n)]


def _engine(compress=True, **kw):
    comp = random_compressor(KVCacheLinearDecoupleCompressor, 2, 64, 4) if compress else None
    return LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=128, max_model_len=512,
               device="cpu", enforce_eager=True, enable_compression=compress, compressor=comp,
               compression_backend="mlp", **{"compression_pipeline": "prefill", **kw})


# ------------------------------------------------------------------ compressor failure
def test_compressor_exception_leaves_requests_uncompressed_and_serving():
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    want = _engine(compress=False).generate(_prompts(), sp)
    llm = _engine(compress=True)
    calls = {"n": 0}

    def boom(*a, **k):
        calls["n"] += 1
        raise RuntimeError("injected compressor failure")

    llm.model_runner.compress_kv_cache_batch = boom
    got = llm.generate(_prompts(), sp)
    assert calls["n"] >= 1 and llm.stats.compress_failures >= 1
    assert isinstance(llm.last_compress_error, RuntimeError)
    # nothing was compressed, so the tokens are those of the uncompressed engine
    assert [o["token_ids"] for o in got] == [o["token_ids"] for o in want]
    llm.scheduler.block_manager.check_invariants()
    assert llm.scheduler.block_manager.num_free_blocks == llm.scheduler.block_manager.num_blocks


def test_compressor_exception_policy_raise():
    llm = _engine(compress=True)
    llm.compression_error_policy = "raise"
    llm.model_runner.compress_kv_cache_batch = lambda *a, **k: (_ for _ in ()).throw(ValueError("injected"))
    for p in _prompts(2):
        llm.add_request(p, SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    with pytest.raises(ValueError):
        llm.step()
    # the lengths the failed call had overwritten are restored
    assert all(s.compression_state is CompressionState.NONE for s in llm.scheduler.running)


# ------------------------------------------------------------------------- cancellation
def test_abort_running_and_waiting_requests_returns_blocks():
    sp = SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True)
    llm = _engine(compress=True, max_num_seqs=2)
    seqs = [llm.add_request(p, sp) for p in _prompts(4)]
    llm.step()                                         # two requests prefilled, two still waiting
    running = list(llm.scheduler.running)
    waiting = list(llm.scheduler.waiting)
    assert len(running) == 2 and len(waiting) == 2
    assert llm.abort_request(running[0].seq_id)
    assert llm.abort_request(waiting[0].seq_id)
    assert not llm.abort_request(running[0].seq_id)    # already gone
    assert not llm.abort_request(10 ** 9)
    while not llm.is_finished():
        llm.step()
    done = [s for s in seqs if s.num_completion_tokens == 16]
    assert len(done) == 2 and llm.stats.aborted == 2
    bm = llm.scheduler.block_manager
    bm.check_invariants()
    assert bm.num_free_blocks == bm.num_blocks


# ---------------------------------------------------------------------------- recovery
def test_recover_requeues_running_requests_and_output_is_unchanged():
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    want = _engine(compress=False).generate(_prompts(), sp)
    llm = _engine(compress=False)
    seqs = [llm.add_request(p, sp) for p in _prompts()]
    for _ in range(5):
        llm.step()
    assert llm.recover() == 4                          # the step "in flight" is abandoned
    bm = llm.scheduler.block_manager
    assert bm.num_free_blocks == bm.num_blocks and not llm.scheduler.running
    while not llm.is_finished():
        llm.step()
    # recompute replays prompt + tokens so far, so greedy outputs are those of an undisturbed run
    assert [s.completion_token_ids for s in seqs] == [o["token_ids"] for o in want]
    assert llm.stats.recoveries == 1


def test_recover_with_compression_pending():
    sp = SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True)
    llm = _engine(compress=True, compression_pipeline="decode")
    seqs = [llm.add_request(p, sp) for p in _prompts(3)]
    llm.step()
    llm.step()
    llm.recover()
    assert not llm._pending
    assert all(s.compression_state is CompressionState.NONE and not s.hold for s in seqs)
    while not llm.is_finished():
        llm.step()
    assert all(s.num_completion_tokens == 6 for s in seqs)
    llm.scheduler.block_manager.check_invariants()


def test_pool_exhaustion_is_reported_not_hung():
    llm = LLM(tiny_llama_config(), kvcache_block_size=16, num_kvcache_blocks=4, max_model_len=512,
              device="cpu", enforce_eager=True)
    llm.add_request(_prompts(1, length=200)[0], SamplingParams(max_tokens=4))
    with pytest.raises(RuntimeError, match="blocks"):
        llm.step()


def test_device_status_code_becomes_exception():
    llm = _engine(compress=False)
    llm.check_device_status()                          # CPU runner: always clean
    llm.model_runner.read_device_status = lambda: 5    # what a peer wait that ran out would leave
    with pytest.raises(DeviceWaitTimeout) as e:
        llm.check_device_status()
    assert e.value.code == 5 and "another GPU" in str(e.value)


# ---------------------------------------------------------------------------- watchdog
def test_step_watchdog_fires_once_and_raises():
    fired = []
    wd = StepWatchdog(0.05, on_expire=lambda label, t: fired.append((label, t)))
    with wd.step("fast"):
        pass
    with pytest.raises(StepDeadlineExceeded):
        with wd.step("slow"):
            time.sleep(0.25)
    with wd.step("fast again"):
        pass
    wd.close()
    assert [f[0] for f in fired] == ["slow"] and fired[0][1] >= 0.05


def test_watchdog_triggers_engine_recovery():
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    llm = _engine(compress=False)
    seqs = [llm.add_request(p, sp) for p in _prompts(2)]
    llm.step()
    wd = StepWatchdog(0.05)
    real_run = llm.model_runner.run

    def stuck_once(batch, is_prefill):
        time.sleep(0.2)                                # a step that overruns (host side only)
        llm.model_runner.run = real_run
        return real_run(batch, is_prefill)

    llm.model_runner.run = stuck_once
    with pytest.raises(StepDeadlineExceeded):
        with wd.step("decode"):
            llm.step()
    llm.recover()
    wd.close()
    calm = StepWatchdog(10.0)                          # generous: the box running the tests may be busy
    while not llm.is_finished():
        with calm.step("step"):
            llm.step()
    calm.close()
    assert all(s.num_completion_tokens == 4 for s in seqs)


# --------------------------------------------------------------------------- heartbeat
def test_heartbeat_detects_silent_and_departed_ranks():
    store = dist.HashStore()
    hbs = [RankHeartbeat(store, r, 3, period_s=0.02, timeout_s=0.2) for r in range(3)]
    time.sleep(0.1)
    assert hbs[0].dead_ranks() == []
    hbs[2].pause()                                     # rank 2 hangs: process alive, no progress
    deadline = time.monotonic() + 3.0
    while time.monotonic() < deadline and hbs[0].dead_ranks() != [2]:
        time.sleep(0.05)
    assert hbs[0].dead_ranks() == [2]
    hbs[1].dead_ranks()                                # first look only records the counter
    time.sleep(0.3)
    with pytest.raises(RankFailure) as e:
        hbs[1].check()
    assert e.value.ranks == [2]
    hbs[2].resume()
    time.sleep(0.1)
    assert hbs[0].dead_ranks() == []
    hbs[1].leave()                                     # an orderly exit is seen at once
    assert hbs[0].dead_ranks() == [1]
    for h in hbs:
        h.close()


def _rank_main(rank, world, port, q):
    """gloo ranks: rank 1 leaves between steps; rank 0 learns of it from the heartbeat before its
    next collective, and a collective entered anyway ends with an error after the short timeout."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20),
                          wait_for_workers=True)
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world,
                            timeout=timedelta(seconds=2))
    hb = RankHeartbeat(dist.PrefixStore("hb", store), rank, world, period_s=0.05, timeout_s=0.5)
    x = torch.ones(4) * (rank + 1)
    dist.all_reduce(x)                                  # step 1: everyone present
    ok_first = bool(torch.allclose(x, torch.full((4,), 3.0)))
    if rank == 1:
        hb.leave()                                      # leaves between steps, nothing in flight
        hb.close()
        q.put(("left", rank, ok_first))
        time.sleep(4.0)                                 # keep the store's peer socket open meanwhile
        return
    deadline = time.monotonic() + 5.0
    dead = []
    while time.monotonic() < deadline and not dead:
        dead = hb.dead_ranks()
        time.sleep(0.05)
    err = None
    t0 = time.monotonic()
    try:                                                # what would happen without the heartbeat
        dist.all_reduce(torch.ones(4))
    except Exception as exc:                            # the short timeout turns a hang into an error
        err = type(exc).__name__
    q.put(("survivor", dead, ok_first, err, time.monotonic() - t0))
    hb.close()


def test_dead_rank_is_detected_by_gloo_survivor():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    msgs = [q.get(timeout=60) for _ in range(2)]
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()                                    # exact child, never a pattern
    left = [m for m in msgs if m[0] == "left"][0]
    surv = [m for m in msgs if m[0] == "survivor"][0]
    assert left[2] and surv[2]                          # the collective before the failure was correct
    assert surv[1] == [1]                               # learnt on the host, before any launch
    assert surv[3] is not None and surv[4] < 15.0       # the orphaned collective errored, it did not hang


# ------------------------------------------------------- device waits that run out (one GPU, nothing faults)
def test_step_raises_when_the_runner_reports_a_status_code():
    """The status word comes back with the sampled tokens; `step()` turns a non-zero code into an exception and
    `recover()` then serves every request."""
    sp = SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True)
    llm = _engine(compress=False)
    seqs = [llm.add_request(p, sp) for p in _prompts(2)]
    llm.step()
    r = llm.model_runner
    real = r.run

    def run_with_timeout(batch, is_prefill, **kw):
        out = real(batch, is_prefill, **kw)
        r.last_status = 5
        return out

    r.run = run_with_timeout
    with pytest.raises(DeviceWaitTimeout) as e:
        llm.step()
    assert e.value.code == 5 and r.last_status == 0
    r.run = real
    assert llm.recover() == 2
    while not llm.is_finished():
        llm.step()
    assert all(s.num_completion_tokens == 4 for s in seqs)


def test_controller_timings_agree_across_ranks(monkeypatch):
    """Under tensor parallelism the controller is fed the slowest rank's step time, and a compression only
    counts as finished when it has finished on every rank."""
    import torch.distributed as dist
    from fastcache_b200.parallel import tp as tpmod
    llm = _engine(compress=False)
    other = [7.0, -0.0, -1.0, 0.0, 2.5]           # the peer: slower step, first compression still running

    def fake_all_reduce(t, op=None, group=None):
        assert op == dist.ReduceOp.MAX
        t.copy_(torch.maximum(t, torch.tensor(other, dtype=t.dtype)))

    monkeypatch.setattr(tpmod, "get_tp_size", lambda: 2)
    monkeypatch.setattr(dist, "all_reduce", fake_all_reduce)
    ms, done, c_ms = llm._agree_on_timings(5.0, [True, True], [1.0, 2.0])
    assert ms == 7.0 and done == [False, True] and c_ms[1] == 2.5


@pytest.mark.gpu
def test_peer_wait_runs_out_on_a_flag_that_nothing_posts():
    """One GPU plays rank 0 of two: the second rank's flag words are local memory that nobody writes.  With the
    wait limit set to 5 ms the fused all-reduce returns, the status word reads `timeout waiting for a flag
    written by another GPU`, and the engine's next step raises `DeviceWaitTimeout`.  Nothing traps or hangs:
    the wait is bounded and the context stays usable."""
    from fastcache_b200 import ops
    e = ops.ext()
    dev = torch.device("cuda", 0)
    H, T = 1024, 4
    bufs = [torch.zeros(2, 64, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]      # [rank][rows][H]
    flags = torch.zeros(2, 512 * 8, dtype=torch.int32, device=dev)
    status = e.status_tensor(0)
    e.read_status(0)
    try:
        e.comm_init(0, 2, [bufs[0][0].data_ptr(), bufs[0][1].data_ptr()],
                    [bufs[1][0].data_ptr(), bufs[1][1].data_ptr()],
                    [flags[0].data_ptr(), flags[1].data_ptr()], 0, 0, 0)
        e.set_wait_limit_us(0, 5000)
        resid = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        w = torch.ones(H, dtype=torch.bfloat16, device=dev)
        t0 = time.perf_counter()
        e.allreduce_add_rmsnorm(0, resid, w, 1e-6, False, status)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 2.0                  # the built-in limit would be 10 s
        assert int(flags[1].view(512, 8)[:T, 0].min()) == 1    # rank 0 posted its arrival to "rank 1"
        # the engine learns of it with the next tokens it reads back
        llm = LLM(tiny_llama_config(head_dim=128, hidden_size=512), device="cuda:0", kvcache_block_size=16,
                  num_kvcache_blocks=32, max_model_len=256, enforce_eager=True)
        llm.add_request(_prompts(1, length=20)[0], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
        with pytest.raises(DeviceWaitTimeout) as err:
            llm.step()
        assert err.value.code == 5
        assert e.read_status(0) == 0                           # cleared by the engine
        assert llm.recover() == 1
        while not llm.is_finished():
            llm.step()
        llm.exit()
    finally:
        e.set_wait_limit_us(0, 0)
        e.read_status(0)
        e.comm_shutdown()
