"""Host side of the row-sharded path on CPU: two gloo ranks each compute their row
interval of a quantized mat-vec with the oracle's kernels and join the intervals with
an all-gather, as the GPU ranks do; the joined vector must equal the unsharded product
bit for bit (the reference's lane-count invariance, tests/kernel/matmul_tests.cpp:597-724),
and the greedy head's candidate merge must keep the lowest-row tie rule."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port_no, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    import emel_cpp_b200 as eb
    from emel_cpp_b200 import llama as el
    from oracle import bindings as ob
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    port = ob.port()
    for t, k, m in ((eb.Q4_K, 512, 64), (eb.Q6_K, 256, 48), (eb.Q8_0, 128, 40)):
        rng = np.random.Generator(np.random.PCG64(11))          # same tensors on both ranks
        w = rng.standard_normal((m, k), dtype=np.float32) * np.float32(0.05)
        x = rng.standard_normal(k, dtype=np.float32)
        blocks = port.encode_rows(t, w, k, m)
        y_full = np.zeros(m, np.float32)
        assert port.mul_mat(ob.mul_mat_op(blocks, t, k, m, x, 1, y_full))
        row0, rows = el.shard_rows(m, rank, world)
        rb = eb.row_bytes(t, k)
        mine = np.ascontiguousarray(blocks.reshape(-1)[row0 * rb:(row0 + rows) * rb])   # contiguous byte range of the tensor
        y_mine = np.zeros(rows, np.float32)
        assert port.mul_mat(ob.mul_mat_op(mine, t, k, rows, x, 1, y_mine))
        parts = [torch.zeros(rows) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(y_mine))
        joined = torch.cat(parts).numpy()
        assert np.array_equal(joined, y_full), (t, float(np.abs(joined - y_full).max()))
        # greedy head: per-rank winner {value, global row}, then highest value / lowest row
        best = int(np.argmax(y_mine))
        pair = torch.tensor([float(y_mine[best]), float(row0 + best)], dtype=torch.float64)
        pairs = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(pairs, pair)
        assert el.merge_argmax_pairs([(float(p[0]), int(p[1])) for p in pairs]) == int(np.argmax(y_full))
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()


def test_two_gloo_ranks_join_row_intervals(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_plan():
    from emel_cpp_b200 import llama as el
    assert el.shard_rows(4096, 3, 8) == (1536, 512)
    with pytest.raises(ValueError):
        el.shard_rows(10, 0, 4)
    full = el.matrix_shapes(el.config(32, 4096, 32, 8, 128, 14336, 128256, 64))
    part = el.matrix_shapes(el.config(32, 4096, 32, 8, 128, 14336, 128256, 64, shard_rank=5, shard_count=8))
    assert part[el.TOKEN_EMBD] == full[el.TOKEN_EMBD]
    for role in (el.ATTN_Q, el.ATTN_K, el.ATTN_V, el.ATTN_OUT, el.FFN_GATE, el.FFN_UP, el.FFN_DOWN, el.OUTPUT):
        assert part[role] == (full[role][0], full[role][1] // 8)
    # ties: highest value, then lowest row, whatever the rank order
    assert el.merge_argmax_pairs([(1.0, 900), (2.0, 70), (2.0, 12), (0.5, 3)]) == 12
