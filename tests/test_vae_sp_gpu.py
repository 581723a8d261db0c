"""Time-sharded VAE decode on 2 GPUs (NCCL halo exchange + GroupNorm all-reduce) against the single-GPU
decode. Each rank decodes a slab of latent frames; the concatenation must match the unsharded result up to
the order of the GroupNorm sums (fp64, so in practice bit for bit). Skipped with fewer than two GPUs."""
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
    from rapid_h3_b200 import _lib, vae
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dec = vae.VAEDecoder(seed=1, widths=(128, 64, 64), blocks_per_stage=1, device=f"cuda:{rank}")
        g = torch.Generator().manual_seed(5)
        latent = torch.randn(1, 16, 5, 3, 4, generator=g).to(torch.bfloat16).cuda()
        ref = dec.decode(latent)
        sp = vae.TimeShards(latent.shape[2])
        mine = dec.decode(latent[:, :, sp.t0:sp.t1].contiguous(), sp=sp)
        _lib.check_status()
        # frames of the output owned by this rank: latent frames [t0, t1) -> 4*t0 - 3 .. 4*t1 - 4 (rank 0 from 0)
        lo = 0 if sp.t0 == 0 else 4 * sp.t0 - 3
        hi = 4 * sp.t1 - 3
        want = ref[:, :, lo:hi]
        rel = ((mine.float() - want.float()).norm() / want.float().norm()).item()
        ret[rank] = (tuple(mine.shape) == tuple(want.shape), rel)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_rank_decode_equals_single_gpu_decode():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in (0, 1):
        ok_shape, rel = ret[r]
        assert ok_shape and rel <= 2e-3, dict(ret)
