"""The N>1 host logic on CPU: sharding rules, and the KV-range exchange (all-gather of partial
softmax states, then merge) run as two gloo ranks against the unsharded CPU result."""
import os
import socket

import numpy as np
import pytest

from mugen_b200 import sharding, synth


def test_shard_batch_covers_everything_once():
    for n, w in [(64, 1), (64, 8), (65, 8), (3, 4), (128, 2)]:
        got = [i for r in range(w) for i in sharding.shard_batch(n, w, r)]
        assert got == list(range(n))
        sizes = [len(sharding.shard_batch(n, w, r)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1


def test_shard_by_load_balances_ragged_batches():
    lens = synth.ragged_lengths(42, 128, 256, 32768)
    for w in (2, 4, 8):
        parts = sharding.shard_by_load(lens, w)
        assert sorted(i for p in parts for i in p) == list(range(128))
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) <= 1.1 * sum(lens) / w


def test_kv_range_slices_are_page_aligned_and_cover():
    for S, w in [(131072, 8), (131072, 2), (1000, 4), (63, 4), (64 * 9 + 17, 3)]:
        sl = sharding.kv_range_slices(S, w)
        assert sl[0][0] == 0 and sl[-1][1] == S
        for (a, b), (c, d) in zip(sl, sl[1:]):
            assert b == c and b % 64 == 0 or b == S
        assert all(b >= a for a, b in sl)


def _worker(rank, world, port, q, result):
    import torch
    import torch.distributed as dist
    from oracle import binding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ora = binding.oracle()
        H, S, dt = 8, 64 * 5 + 40, synth.DT_F16
        case = synth.make_layer_case(321, H, [S], dt)
        a, b = sharding.kv_range_slices(S, world)[rank]
        part = ora.partial(case.q[0], case.caches[0], a, b, case.w_uk, synth.W_F16, H, dt)
        part[:, 0] *= np.log2(np.e)                       # the exchanged maximum is in the log2 domain
        if b == a:
            part[:] = 0
            part[:, 0] = -np.inf
        mine = torch.from_numpy(part.reshape(1, H, sharding.PART).copy())
        gathered = torch.zeros((world, 1, H, sharding.PART), dtype=torch.float32)
        dist.all_gather_into_tensor(gathered.view(-1, H, sharding.PART), mine)
        o_c = sharding.merge_partials_reference(gathered.numpy())[0]
        full = ora.partial(case.q[0], case.caches[0], 0, S, case.w_uk, synth.W_F16, H, dt)
        want = full[:, 2:] / full[:, 1:2]
        err = float(np.abs(o_c - want).max())
        # W_UV on the merged state equals the unsharded attention output
        out = (o_c[:, None, :] * case.w_uv_f32.reshape(H, 128, 512)).sum(-1)
        ref = synth.from_bits(ora.attention(case.q[0], case.caches[0], S, case.w_uk, case.w_uv, synth.W_F16, H, dt), dt)
        result.put((rank, err, float(np.abs(out - ref).max())))
    finally:
        dist.destroy_process_group()


def _absent_rank_worker(rank, world, port, result):
    """Ranks 0..world-2 reach the all-gather of a step; the last rank joined the group but never makes the call
    (it stands for a process that hung or died between steps, with nothing of its own in flight)."""
    import datetime
    import time

    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    H = 4
    mine = torch.full((1, H, sharding.PART), float(rank))
    gathered = torch.zeros((world, 1, H, sharding.PART))
    # one healthy exchange first: the group works
    dist.all_gather_into_tensor(gathered.view(-1, H, sharding.PART), mine)
    ok_first = bool((gathered[:, 0, 0, 0] == torch.arange(world, dtype=torch.float32)).all())
    if rank == world - 1:
        result.put((rank, ok_first, "absent", 0.0))
        result.close()
        result.join_thread()                               # the queue's feeder thread must flush before _exit
        time.sleep(12)                                     # never arrives at the second exchange
        os._exit(0)
    t0 = time.time()
    try:
        dist.all_gather_into_tensor(gathered.view(-1, H, sharding.PART), mine)
        outcome = "completed"
    except Exception as e:                                 # the process group's timeout, reported on the host
        outcome = "gave up: " + type(e).__name__
    result.put((rank, ok_first, outcome, time.time() - t0))
    result.close()
    result.join_thread()
    os._exit(0)                                            # the group is broken: no orderly teardown to wait for


def test_a_rank_that_never_reaches_the_all_gather_is_detected_by_timeout():
    """Failure detection without touching a GPU: the exchange step of the KV-range mode is a host-issued
    collective, so a missing rank shows as a timeout error on the surviving ranks' host threads (seconds, set
    on the process group), never as a device-side spin."""
    import torch.multiprocessing as mp
    world = 3
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    procs = [ctx.Process(target=_absent_rank_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    got = sorted(result.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    for rank, ok_first, outcome, waited in got:
        assert ok_first, rank
        if rank == world - 1:
            assert outcome == "absent"
        else:
            assert outcome.startswith("gave up"), (rank, outcome)
            assert 1.0 < waited < 30.0, (rank, waited)


@pytest.mark.parametrize("world", [2, 3])
def test_kv_range_exchange_over_gloo(world):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q, result = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, result)) for r in range(world)]
    for p in procs:
        p.start()
    got = [result.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_state, err_out in got:
        assert err_state < 1e-5, (rank, err_state)
        assert err_out < 2e-3, (rank, err_out)
