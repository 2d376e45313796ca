"""Batch-sharded training on two CPU ranks (gloo): sharded grads + one all-reduce
equal the single-process full-batch grads."""

from __future__ import annotations

import os
import socket
import sys
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import REPO


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _make_layer():
    from gru_triton_b200 import GRULayer, QuantizerConfig, QuantRecipe, StructureConfig
    torch.manual_seed(5)
    rec = QuantRecipe(weight=QuantizerConfig(bits=32, axis=0), input_act=QuantizerConfig(bits=32),
                      hidden=QuantizerConfig(bits=32))
    return GRULayer(12, 16, rec, gate_layout="fused", structure_hidden=StructureConfig(kind="diagonal"))


def _worker(rank, world, port, out_path):
    sys.path.insert(0, REPO)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from gru_triton_b200.data_parallel import (GradBucket, OverlappedReducer, hidden_then_input_buckets,
                                               shard_batch)
    layer = _make_layer()
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(6, 5, 12, generator=gen)            # B = 5: uneven shards (3 + 2)
    h0 = torch.randn(5, 16, generator=gen)
    out, _ = layer(shard_batch(x, rank, world, 1), shard_batch(h0, rank, world, 0))
    out.sum().backward()
    params = [p for p in layer.parameters()]
    GradBucket(params).all_reduce()
    one_bucket = [p.grad.clone() for p in params]
    # the same step with two buckets, each reduced from the hook of its last gradient
    buckets = hidden_then_input_buckets(layer)
    assert len(buckets[0]) and len(buckets[1]) and len(buckets[0]) + len(buckets[1]) == len(params)
    for in_place in (True, False):                      # coalesced in-place collective / flat buckets
        red = OverlappedReducer(buckets, in_place=in_place)
        for _ in range(2):                              # twice: the counters re-arm
            layer.zero_grad(set_to_none=True)
            out, _ = layer(shard_batch(x, rank, world, 1), shard_batch(h0, rank, world, 0))
            out.sum().backward()
            red.finish()
            for a, p in zip(one_bucket, params):
                assert torch.equal(a, p.grad)
        red.remove()
    if rank == 0:
        torch.save(one_bucket, out_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_sharded_grads_match_full_batch():
    from gru_triton_b200.data_parallel import shard_bounds
    assert [shard_bounds(5, r, 2) for r in range(2)] == [(0, 3), (3, 5)]
    assert [shard_bounds(4096, r, 8) for r in range(8)][-1] == (3584, 4096)
    ctx = mp.get_context("spawn")
    port = _free_port()
    out_path = os.path.join(tempfile.mkdtemp(), "grads.pt")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out_path)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    got = torch.load(out_path)
    layer = _make_layer()
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(6, 5, 12, generator=gen)
    h0 = torch.randn(5, 16, generator=gen)
    out, _ = layer(x, h0)
    out.sum().backward()
    for g, p in zip(got, layer.parameters()):
        assert (g - p.grad).abs().max().item() < 1e-5


def test_bucket_split_follows_the_backward_order():
    """hidden_then_input_buckets: the hidden path's parameters (finished by the scan backward) first,
    the input projection's second, for every hidden kind; nothing lost, nothing twice."""
    from gru_triton_b200 import GRULayer, QuantizerConfig, QuantRecipe, StructureConfig
    from gru_triton_b200.data_parallel import hidden_then_input_buckets
    rec = QuantRecipe(weight=QuantizerConfig(bits=32, axis=0), input_act=QuantizerConfig(bits=32),
                      hidden=QuantizerConfig(bits=32))
    for st in (None, StructureConfig(kind="diagonal"), StructureConfig(kind="monarch", nblocks=4),
               StructureConfig(kind="butterfly")):
        layer = GRULayer(16, 16, rec, gate_layout="fused", structure_hidden=st)
        names = {id(p): n for n, p in layer.named_parameters()}
        hidden, rest = hidden_then_input_buckets(layer)
        assert len(hidden) == 6 and len(rest) == 6
        assert {id(p) for p in hidden} | {id(p) for p in rest} == set(names)
        assert all(("_h" in names[id(p)]) or ("struct_Wh" in names[id(p)]) for p in hidden)
        assert all(("W_i" in names[id(p)]) or ("b_i" in names[id(p)]) for p in rest)
