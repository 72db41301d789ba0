"""One rank of the row-sharded checks (launched by tests/test_gpu_sharded.py through
torch.distributed.run, one process per GPU).

Each rank builds, on its own GPU, (a) the unsharded decoder session over the full
seeded matrices and (b) the sharded session bound to its row interval of the same
bytes, and requires identical results: logits and greedy ids bit for bit with the
reference-order attention, ids identical and logits within the attention tolerance
with the split-KV attention.  It also joins a row-sliced op_mul_mat through
emelb_all_gather_rows and compares it with the unsliced call, which is the reference's
own lane-count invariance test (tests/kernel/matmul_tests.cpp:597-724) across GPUs.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import emel_cpp_b200 as eb  # noqa: E402
from emel_cpp_b200 import llama as el  # noqa: E402

CFG = dict(n_layer=3, n_embd=2048, n_head=16, n_head_kv=4, head_dim=128, n_ff=4096, n_vocab=4096, n_ctx=64)


def build(be, alloc_be, cfg_kw, rank, world, buffers):
    cfg = el.config(shard_rank=rank, shard_count=world, **cfg_kw)
    sess = el.Session(be, cfg)
    full = el.matrix_shapes(el.config(**cfg_kw))
    for layer, role, t in buffers["order"]:
        d = buffers[(layer, role)]
        if role in (el.OUTPUT_NORM, el.ATTN_NORM, el.FFN_NORM):
            assert sess.bind_norm(layer, role, d), sess.last_error
            continue
        k, m = full[role]
        row0 = 0 if role == el.TOKEN_EMBD or world == 1 else el.shard_rows(m, rank, world)[0]
        assert sess.bind_matrix(layer, role, d + row0 * eb.row_bytes(t, k), t), (layer, role, sess.last_error)
    return sess


def idf0_first(results):
    return results[("full", 0)][1][0]


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    be_full, be_shard = eb.Backend(local), eb.Backend(local)
    box = [eb.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    assert be_shard.comm_init(rank, world, box[0]), be_shard.last_error

    # the same seeded tensors on every rank
    shapes = el.matrix_shapes(el.config(**CFG))
    buffers, order, seed = {}, [], 100
    def matrix(layer, role, t, sigma):
        nonlocal seed
        k, m = shapes[role]
        d = be_full.alloc(m * eb.row_bytes(t, k))
        assert be_full.synth_fill(d, t, m * k, seed, sigma, 0), be_full.last_error
        seed += 1
        buffers[(layer, role)] = d
        order.append((layer, role, t))
    def norm(layer, role):
        nonlocal seed
        d = be_full.alloc(4 * CFG["n_embd"])
        w = (1.0 + 0.1 * np.random.Generator(np.random.PCG64(seed)).standard_normal(CFG["n_embd"])).astype(np.float32)
        seed += 1
        assert be_full.to_device(d, w)
        buffers[(layer, role)] = d
        order.append((layer, role, eb.F32))
    matrix(-1, el.TOKEN_EMBD, eb.Q4_K, 1.0)
    norm(-1, el.OUTPUT_NORM)
    matrix(-1, el.OUTPUT, eb.Q6_K, 0.05)
    for l in range(CFG["n_layer"]):
        norm(l, el.ATTN_NORM)
        norm(l, el.FFN_NORM)
        for role in (el.ATTN_Q, el.ATTN_K, el.ATTN_V, el.ATTN_OUT, el.FFN_GATE, el.FFN_UP):
            matrix(l, role, eb.Q4_K, 0.05)
        # layers 0 and 1 qualify for joins inside their kernels (K-quant products), layer 2 (Q8_0) takes a join kernel each
        matrix(l, el.FFN_DOWN, (eb.Q6_K, eb.Q4_K, eb.Q8_0)[l % 3], 0.05)
    buffers["order"] = order
    assert be_full.sync()

    prompt = np.random.Generator(np.random.PCG64(7)).integers(0, CFG["n_vocab"], size=9).tolist()
    results = {}
    # sharded sessions walk the prompt token by token; the unsharded one is held to the same walk here so that
    # the comparison is about sharding alone (the batched prompt path has its own tests)
    for name, be, r, g in (("full", be_full, 0, 1), ("shard", be_shard, rank, world), ("shard-peer", be_shard, rank, world),
                           ("shard-peer-unfused", be_shard, rank, world)):
        for mode in (2, 0):
            be.set_attention_mode(mode)
            sess = build(be, be_full, CFG, r, g, buffers)
            assert sess.set_prefill_batch(0)
            if name.startswith("shard-peer"):       # joins by peer stores instead of NCCL all-gathers
                assert sess.set_join_fusion(name == "shard-peer")
                handles = [None] * world
                dist.all_gather_object(handles, sess.exchange_export())
                assert sess.exchange_attach(handles), sess.last_error
                dist.barrier()             # every rank has mapped its peers before anybody's first join
            assert sess.prefill(prompt[:-1], 0), sess.last_error
            logits = sess.decode(prompt[-1], len(prompt) - 1, want_logits=True)
            ids = sess.generate(prompt[-1], len(prompt) - 1, 12)
            ids_host = [sess.decode(prompt[-1], len(prompt) - 1)]
            results[(name, mode)] = (logits, list(ids), ids_host)
            assert be.sync(), "a bounded device wait ran out"
            dist.barrier()                 # nobody unmaps an arena a peer may still write to
            assert sess.exchange_detach()
            dist.barrier()                 # nobody frees an arena a peer still maps
            sess.close()
    lf, idf, hf = results[("full", 2)]
    ls, ids_, hs = results[("shard", 2)]
    assert np.array_equal(lf, ls), float(np.abs(lf - ls).max())
    assert idf == ids_ and hf == hs and hf[0] == idf[0], (idf, ids_, hf, hs)
    lp, idp, hp = results[("shard-peer", 2)]
    assert np.array_equal(lf, lp) and idf == idp and hf == hp, (float(np.abs(lf - lp).max()), idf, idp)
    assert results[("shard-peer", 0)][1][0] == idf0_first(results)
    # the joins inside the kernels and the join kernels move the same floats: identical logits and ids
    for mode in (2, 0):
        la, ia, ha = results[("shard-peer", mode)]
        lb, ib, hb = results[("shard-peer-unfused", mode)]
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and ia == ib and ha == hb, (mode, float(np.abs(la - lb).max()))
    lf0, idf0, _ = results[("full", 0)]
    ls0, ids0, _ = results[("shard", 0)]
    assert float(np.abs(lf0 - ls0).max()) <= 1e-3
    assert idf0[0] == ids0[0]
    assert float(np.abs(lf0 - results[("shard-peer", 0)][0]).max()) <= 1e-3

    # batched prompt path: the sharded session processes the prompt in token batches too (row intervals of every
    # product joined by NCCL); per head and per row it runs the same kernels on the same numbers as the
    # unsharded session, so the logits that follow are bit-identical
    long_prompt = np.random.Generator(np.random.PCG64(11)).integers(0, CFG["n_vocab"], size=51).tolist()
    batched = {}
    for name, be, r, g in (("full", be_full, 0, 1), ("shard", be_shard, rank, world)):
        be.set_attention_mode(0)
        sess = build(be, be_full, CFG, r, g, buffers)
        assert sess.set_prefill_batch(24)              # 50 prompt tokens = 24 + 24 + 2
        l0 = be.diagnostics()["kernel_launches"]
        assert sess.prefill(long_prompt[:-1], 0), sess.last_error
        launches = be.diagnostics()["kernel_launches"] - l0
        assert launches < 50 * 10, launches            # batches, not 50 token steps of 15+ launches
        batched[name] = sess.decode(long_prompt[-1], 50, want_logits=True)
        assert be.sync()
        dist.barrier()
        sess.close()
    assert np.array_equal(batched["full"].view(np.uint32), batched["shard"].view(np.uint32)), \
        float(np.abs(batched["full"] - batched["shard"]).max())

    # several sequences stepped together in a sharded session (joins of the batch tensors by NCCL): every sequence
    # gets the ids it gets alone in the same session
    be_shard.set_attention_mode(0)
    sess = build(be_shard, be_full, CFG, rank, world, buffers)
    assert sess.set_sequences(3), sess.last_error
    firsts, poss, alone = [], [], []
    for j in range(3):
        pj = np.random.Generator(np.random.PCG64(30 + j)).integers(0, CFG["n_vocab"], size=7 + 2 * j).tolist()
        assert sess.select_sequence(j) and sess.prefill(pj[:-1], 0), sess.last_error
        firsts.append(pj[-1])
        poss.append(len(pj) - 1)
    for j in range(3):
        assert sess.select_sequence(j)
        alone.append(list(sess.generate(firsts[j], poss[j], 6)))
    together = sess.generate_batch(firsts, poss, 6)
    for j in range(3):
        assert list(together[:, j]) == alone[j], (j, list(together[:, j]), alone[j])
    assert be_shard.sync()
    dist.barrier()
    sess.close()

    # op level: each rank runs its row slice of one op_mul_mat, then the join
    k, m, n = 2048, 4096, 3
    w = be_full.alloc(m * eb.row_bytes(eb.Q4_K, k))
    assert be_full.synth_fill(w, eb.Q4_K, m * k, 900, 0.05, 0)
    x = be_full.alloc(4 * k * n)
    assert be_full.synth_fill(x, eb.F32, k * n, 901, 1.0, 0)
    y_full, y_join = be_full.alloc(4 * m * n), be_shard.alloc(4 * m * n)
    assert be_full.mul_mat(eb.mul_mat_op(w, eb.Q4_K, k, m, x, n, y_full)), be_full.last_error
    assert be_full.sync()
    op = eb.mul_mat_op(w, eb.Q4_K, k, m, x, n, y_join)
    sl, row0, rows = eb.row_slice(op, rank, world)
    assert rows == m // world and row0 == rank * rows
    assert be_shard.mul_mat(sl), be_shard.last_error
    assert be_shard.all_gather_rows(y_join, rows, n), be_shard.last_error
    assert be_shard.sync()
    a, b = np.zeros(m * n, np.float32), np.zeros(m * n, np.float32)
    assert be_full.to_host(a, y_full) and be_shard.to_host(b, y_join)
    assert np.array_equal(a, b)

    be_shard.comm_destroy()
    be_shard.close()
    be_full.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"SHARD_OK rank {rank}", flush=True)


if __name__ == "__main__":
    main()
