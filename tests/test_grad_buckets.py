"""Gradient buckets and the per-bucket shard table of the fused data-parallel path (host logic, CPU):
the arena layout, who owns which slice, and optimizer state moving between rank counts."""
import os
import subprocess
import sys

import pytest
import torch

from allie_b200.data import UCITokenizer
from allie_b200.models import initialize_model
from allie_b200.models.engine import arena_layout, bucket_of
from allie_b200.parallel.nvl import ShardLayout, shard_bounds

HERE = os.path.dirname(os.path.abspath(__file__))


def _model(n_layer=5, **kw):
    tok = UCITokenizer(max_length=64, vocab_size_multiple_of=128)
    torch.manual_seed(0)
    return initialize_model(tok, "gpt2", use_control_token=True, use_regression_head=True, n_layer=n_layer,
                            n_embd=32, n_head=1, n_positions=64, **kw)


def test_buckets_follow_the_order_in_which_backward_finishes_them():
    lay = arena_layout(_model(5), n_layer=5, layers_per_bucket=2)
    assert len(lay["buckets"]) == 3
    where = {n: next(b for b, bk in enumerate(lay["buckets"]) if bk[0] <= o < bk[3]) for n, o in lay["offsets"].items()}
    for n, b in where.items():
        assert b == bucket_of(n, 5, 2), n
    # last blocks + final norm + heads first, embeddings with block 0 last
    assert where["model.model.transformer.h.4.mlp.c_fc.weight"] == 0
    assert where["model.model.transformer.ln_f.weight"] == 0 and where["value_head.0.weight"] == 0
    assert where["model.model.transformer.h.2.attn.c_attn.bias"] == 1
    assert where["model.model.transformer.wte.weight"] == 2 and where["model.model.transformer.h.0.ln_1.weight"] == 2
    # buckets tile [0, sync_end) with nothing in between, every boundary 64-element aligned
    end = 0
    for start, half_end, decay_end, stop in lay["buckets"]:
        assert start == end and start <= half_end <= decay_end <= stop
        assert all(x % 64 == 0 for x in (start, half_end, decay_end, stop))
        end = stop
    assert end == lay["sync_end"] == lay["total"]
    # inside a bucket: GEMM weights, then weight-decayed parameters read as fp32 (the heads), then the rest
    b0 = lay["buckets"][0]
    o = lay["offsets"]
    assert o["model.model.transformer.h.4.mlp.c_fc.weight"] < b0[1]
    assert b0[1] <= o["value_head.0.weight"] < b0[2] and b0[1] <= o["time_head.0.weight"] < b0[2]
    assert b0[2] <= o["model.model.transformer.ln_f.weight"] < b0[3]
    assert b0[2] <= o["value_head.0.bias"] < b0[3]
    # the optimizer ranges cover everything once and carry the right decay flag
    covered = 0
    for s, e, decays in lay["regions"]:
        assert e > s
        covered += e - s
        for n, off in o.items():
            if s <= off < e:
                assert (n in lay["decay_names"]) == decays, n
    assert covered == lay["total"]


def test_one_bucket_layout_keeps_two_optimizer_ranges():
    lay = arena_layout(_model(3), n_layer=3, layers_per_bucket=None)
    assert len(lay["buckets"]) == 1 and len(lay["regions"]) == 2
    assert lay["regions"][0][2] is True and lay["regions"][1][2] is False


def test_every_rank_owns_one_slice_of_every_bucket():
    buckets = [(0, 640, 704, 1024), (1024, 1024 + 4096, 1024 + 4096, 1024 + 4160), (5184, 5184, 5184, 5184 + 64)]
    for world in (1, 2, 3, 4, 8):
        lay = ShardLayout(buckets, world)
        owner = torch.full((lay.end,), -1, dtype=torch.int64)
        for r in range(world):
            m_expect = 0
            for (o, n, m), bk in zip(lay.slices(r), buckets):
                assert m == m_expect and o % 64 == 0 and n % 4 == 0
                assert bk[0] <= o and o + n <= bk[-1]
                assert (owner[o:o + n] == -1).all()
                owner[o:o + n] = r
                m_expect += n
            assert lay.shard_numel(r) == m_expect
        assert (owner >= 0).all()
        # nobody owns much more than 1/world of a bucket
        for bk in buckets:
            assert max(shard_bounds(bk[-1] - bk[0], world, r)[1] for r in range(world)) <= -(-(bk[-1] - bk[0]) // world) + 63


def test_state_sharded_over_eight_ranks_loads_into_one_and_two():
    lay_m = arena_layout(_model(4), n_layer=4, layers_per_bucket=1)
    buckets = lay_m["buckets"]
    full = torch.randn(lay_m["sync_end"])
    eight = ShardLayout(buckets, 8)
    shards8 = [eight.extract(full, r) for r in range(8)]
    assert sum(s.numel() for s in shards8) == full.numel()
    again = eight.assemble(shards8)                       # what a checkpoint written by 8 ranks holds
    assert torch.equal(again, full)
    for world in (1, 2):
        lay = ShardLayout(buckets, world)
        shards = [lay.extract(again, r) for r in range(world)]     # what each rank keeps after loading
        assert torch.equal(lay.assemble(shards), full)
        back = torch.zeros_like(full)
        for r, s in enumerate(shards):
            lay.place(s, r, back)
        assert torch.equal(back, full)


def test_too_many_buckets_are_refused():
    with pytest.raises(AssertionError):
        ShardLayout([(i * 64, i * 64 + 64, i * 64 + 64, i * 64 + 64) for i in range(33)], 2)


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from allie_b200.parallel.nvl import ShardLayout
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
buckets = [(0, 640, 704, 1024), (1024, 5120, 5120, 5184), (5184, 5184, 5184, 5248)]
lay = ShardLayout(buckets, world)
torch.manual_seed(3)
full = torch.randn(lay.end)
mine = lay.extract(full, rank)
out = torch.zeros(lay.end)
lay.all_gather(mine, rank, out)
assert torch.equal(out, full), "all_gather"
dst = torch.zeros(lay.end) if rank == 0 else None
lay.gather(mine, rank, dst, dst=0)
if rank == 0:
    assert torch.equal(dst, full), "gather"
dist.barrier()
dist.destroy_process_group()
print("ok", rank)
"""


def test_shards_gather_across_gloo_ranks(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    env = dict(os.environ)
    env.pop("RANK", None)
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3",
                          "--master-addr", "127.0.0.1", "--master-port", "29641", str(script), os.path.dirname(HERE)],
                         env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
