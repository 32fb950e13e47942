"""Two-GPU checks (skipped on a one-GPU box): a KV-range-sharded sequence whose partial states
travel through an NCCL all-gather, and a batch sharded by sequence, both against the CPU checker."""
import os
import socket

import numpy as np
import pytest

from mugen_b200 import sharding, synth

pytestmark = pytest.mark.gpu
ROPE = dict(rope_theta=10000.0, rope_scaling_factor=40.0, rope_original_ctx=4096, rms_norm_eps=1e-6)


def _rank_main(rank, world, port, result):
    import torch
    import torch.distributed as dist
    from mugen_b200.mla import MlaContext
    from oracle import binding
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ora = binding.oracle()
        H, dt, S = 128, synth.DT_BF16, 64 * 37 + 11
        case = synth.make_layer_case(555, H, [S], dt)
        dev = lambda bits: torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()
        # ---- KV-range: this rank holds rows [a, b) of the one sequence
        a, b = sharding.kv_range_slices(S, world)[rank]
        ctx = MlaContext(n_layers=1, n_heads=H, dtype=dt, n_pages=64, max_seqs=1, max_seq_len=4096,
                         max_position=8192, device=rank, **ROPE)
        ctx.set_layer_weights(0, case.w_uk, case.w_uv, case.w_type, case.norm_w)
        s = ctx.seq_create()
        ctx.seq_set_base(s, a)
        if b > a:
            ctx.write_rows(0, s, 0, dev(case.caches[0][a:b]))
        ctx.advance_seq_len(s, b - a)
        owner = rank == world - 1
        partial = torch.zeros((1, H, sharding.PART), dtype=torch.float32, device="cuda")
        gathered = torch.zeros((world, 1, H, sharding.PART), dtype=torch.float32, device="cuda")
        out = torch.zeros((1, H, 128), dtype=torch.int16, device="cuda")
        ctx.step_begin([s], [1 if owner else 0])
        ctx.step_append(0, dev(case.kv_a))
        sharding.kv_range_attend(ctx, 0, dev(case.q), partial, gathered, out)
        ctx.step_end()
        new_row = ora.append_rows(case.kv_a, [S], case.norm_w, 1e-6, 40.0, 4096, 10000.0, dt)
        full = np.concatenate([case.caches[0], new_row])
        want = ora.attention(case.q[0], full, S + 1, case.w_uk, case.w_uv, case.w_type, H, dt)
        err = synth.error_norms(out.cpu().numpy().view(np.uint16)[0], want, dt, dt)
        assert ctx.status() == 0
        ctx.close()
        dist.barrier()
        result.put((rank, "kv_range", err))
    finally:
        dist.destroy_process_group()


def test_kv_range_over_nccl():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    mpc = mp.get_context("spawn")
    result = mpc.Queue()
    world = 2
    procs = [mpc.Process(target=_rank_main, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    got = [result.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, what, (mx, rl) in got:
        assert mx <= 2e-2 and rl <= 5e-3, (rank, what, mx, rl)
