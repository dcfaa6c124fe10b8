"""Column-parallel linear with the gather done by peer stores, as real ranks: one process per GPU.

Needs two GPUs (skipped otherwise; the single-GPU suite covers the same addressing and flag logic with emulated
ranks run one after the other).  Every rank shards two weights by rows, runs the two gathered linears back to back
for several steps -- the second one waits for the first one's arrivals from all ranks -- in all three forms (stores
fused into the streaming kernel; stores by the tcgen05 path's second kernel; push kernel behind the default kernels) and checks its gathered buffers against
the NCCL all-gather of the same shards (bit-equal for the forms that use the default kernels) and against the
CPU oracle.  No wait may run out.
"""
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker():
    import torch.distributed as dist
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    sys.path.insert(0, ROOT)
    import atlasinfer_b200 as ab
    from atlasinfer_b200 import peer, sharding
    from atlasinfer_b200.integration import atlas_wrappers as aw
    from oracle import atlas_oracle as O
    from tests.util import bits, config_weights, rel_max_err

    m, k, n1, n2, steps = 32, 512, 2048, 512, 6
    o1, o2 = O.quantize(config_weights(n1, k, 61, 0.03)), O.quantize(config_weights(n2, n1, 62, 0.03))
    q1, q2 = ab.QuantizedTensor(*o1), ab.QuantizedTensor(*o2)
    gen = torch.Generator().manual_seed(4)
    xs = [torch.randn(m, k, generator=gen).to(torch.bfloat16) for _ in range(steps)]
    b1 = (torch.randn(n1, generator=gen) * 0.02).half()
    lo1, hi1 = sharding.row_bounds(n1, world, rank, 16)
    lo2, hi2 = sharding.row_bounds(n2, world, rank, 16)
    lay1 = aw.build_kernel_layout(sharding.shard_rows(q1, lo1, hi1).to(dev))
    lay2 = aw.build_kernel_layout(sharding.shard_rows(q2, lo2, hi2).to(dev))
    bias1 = b1[lo1:hi1].to(dev)

    def nccl_gather(y):
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y.contiguous())
        return torch.cat(parts, dim=1)

    arena = peer.PeerArena(1 << 22, dev)
    try:
        for kernel in ("push", "gemm", "stream"):
            g1 = peer.GatheredLinear(arena, lay1, m, torch.bfloat16, bias=bias1, kernel=kernel)
            g2 = peer.GatheredLinear(arena, lay2, m, torch.bfloat16, kernel=kernel)
            for step in range(steps):
                x = xs[step].to(dev)
                g1(x, wait=step > 0)      # a rank may not overwrite g1's buffers before everyone has used them
                g2(g1.out, wait=True)
                g2.wait_for_all()
                torch.cuda.synchronize()
                aw.check_status(dev)
                y1, y2 = g1.out.clone(), g2.out.clone()
                ref1 = O.linear(xs[step], O.dequantize(o1), b1)
                assert rel_max_err(y1, ref1, report=f"{kernel} step {step} layer 1 rank {rank}") < 1e-2
                ref2 = O.linear(y1.cpu(), O.dequantize(o2))
                assert rel_max_err(y2, ref2, report=f"{kernel} step {step} layer 2 rank {rank}") < 1e-2
                if kernel in ("push", "gemm"):
                    want1 = nccl_gather(aw.quantized_linear_forward(x, lay1, bias1))
                    want2 = nccl_gather(aw.quantized_linear_forward(want1, lay2, None))
                    assert torch.equal(bits(y1), bits(want1)) and torch.equal(bits(y2), bits(want2))
                # every rank holds the same gathered bits
                both = [torch.empty_like(y2) for _ in range(world)]
                dist.all_gather(both, y2)
                assert all(torch.equal(bits(b), bits(y2)) for b in both)
                dist.barrier()            # nobody starts the next step's stores while a peer still reads this one's
    finally:
        arena.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok", flush=True)


@pytest.mark.gpu
def test_gathered_linears_on_two_gpus(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.abspath(__file__)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "rank 0 ok" in res.stdout and "rank 1 ok" in res.stdout


if __name__ == "__main__":
    worker()
