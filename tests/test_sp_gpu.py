"""Sequence-parallel step on 2, 4 and 8 GPUs (NCCL) against the single-GPU step: token shards + Ulysses exchange
must reproduce the single-GPU result exactly (every op is row-local or head-local, and the attention statistics
of a head always see its full sequence): with the NCCL all-to-all exchanges, with the exchanges done by the
kernels (stores into peer buffers), and with the two CFG samples side by side on two streams, each with its own
group and buffers. A case is skipped when fewer GPUs are visible than it needs."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    import rapid_h3_b200 as r
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        heads = max(4, world)
        cfg = r.model.H3Config.tiny(n_blocks=2, heads=heads, d_model=128 * heads, mlp_hidden=1024)
        model = r.model.init_weights(r.model.H3Transformer(cfg), seed=2).cuda()
        # 221 tokens: shards of 128 + 93 on two ranks; 587 tokens: ten 64-token blocks over 4 or 8 ranks, the last
        # shard ragged (11 tokens)
        grid, n_audio = ((5, 6, 7), 11) if world <= 2 else ((8, 8, 9), 11)
        inputs = [t.cuda() for t in r.step.make_inputs(cfg, grid, n_audio, 2, 40, seed=3)]
        rt = r.step.H3Runtime(model)
        ref_v, ref_a = rt.step(*inputs)                       # every rank: the whole sequence on its own GPU
        sp = r.sp.Ulysses(grid[0] * grid[1] * grid[2] + n_audio)
        v, a = rt.step(*inputs, sp=sp)
        r._lib.check_status()
        ok = bool(torch.equal(v, ref_v) and torch.equal(a, ref_a))
        # the same step with both exchanges done by the kernels (stores into peer buffers + stream-ordered barriers)
        how = sp.enable_fused(cfg.heads, 128, torch.device("cuda", rank))
        for _ in range(2):  # twice: the exchange buffers are reused from call to call
            v2, a2 = rt.step(*inputs, sp=sp)
        r._lib.check_status()
        ok2 = bool(torch.equal(v2, ref_v) and torch.equal(a2, ref_a))
        # the two CFG samples side by side: a stream, a process group and a set of exchange buffers each
        sps = [r.sp.Ulysses(sp.total, group=dist.new_group(list(range(world)))) for _ in range(2)]
        for u in sps:
            u.enable_fused(cfg.heads, 128, torch.device("cuda", rank))
        streams = [torch.cuda.Stream() for _ in range(2)]
        for _ in range(2):
            v3, a3 = rt.step(*inputs, sp=sps, streams=streams)
        torch.cuda.synchronize()
        r._lib.check_status()
        ok3 = bool(torch.equal(v3, ref_v) and torch.equal(a3, ref_a))
        ret[rank] = (ok, ok2 and ok3, how)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_step_equals_single_gpu_step(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    out = dict(ret)
    print(f"{world} ranks: sharded step == single-GPU step: {[out[r][:2] for r in range(world)]}; peer buffers via {out[0][2]}")
    assert [out[r][:2] for r in range(world)] == [(True, True)] * world, out


@pytest.mark.timeout(300)
def test_fused_exchange_kernels_on_one_rank():
    """World size 1: the scatter kernels write this GPU's own buffers, so their addressing (token rows, head
    groups, q | k | v planes, output ranges) is checked against the unfused step without a second GPU."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(1, _free_port(), ret), nprocs=1, join=True)
    out = dict(ret)
    assert out[0][:2] == (True, True), out
