"""emelb_llama_check_config: the decoder session's configuration guard, run without a device.

A sharded session joins f32 row intervals across ranks in 16-byte units, so a layout whose
per-rank interval is not a multiple of 4 values has to be refused before any kernel sees it."""
import emel_cpp_b200 as eb
from emel_cpp_b200 import llama as el


def cfg(**kw):
    base = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=512, n_vocab=1024, n_ctx=64)
    base.update(kw)
    return el.config(**base)


def test_plain_configurations():
    assert el.check_config(cfg()) == eb.OK
    assert el.check_config(cfg(n_embd=250)) == eb.INVALID_REQUEST          # not a multiple of the K-quant block
    assert el.check_config(cfg(n_head=3)) == eb.INVALID_REQUEST            # query heads per KV head
    assert el.check_config(cfg(rope_dim=63)) == eb.INVALID_REQUEST
    assert el.check_config(cfg(shard_count=0)) == eb.INVALID_REQUEST
    assert el.check_config(cfg(shard_rank=2, shard_count=2)) == eb.INVALID_REQUEST
    assert eb.lib().emelb_llama_check_config(None) == eb.INVALID_REQUEST


def test_sharded_intervals_must_be_whole_and_16_byte_multiples():
    assert el.check_config(cfg(shard_count=2)) == eb.OK
    assert el.check_config(cfg(shard_count=2, shard_rank=1)) == eb.OK
    # 32002 / 2 = 16001 logits per rank: a 4-byte aligned interval, refused
    assert el.check_config(cfg(n_vocab=32002, shard_count=2)) == eb.INVALID_REQUEST
    assert el.check_config(cfg(n_vocab=32008, shard_count=2)) == eb.OK
    # odd head size: 2 heads x 33 dims per rank = 66 values, not a multiple of 4
    assert el.check_config(cfg(head_dim=33, rope_dim=32, shard_count=2)) == eb.INVALID_REQUEST
    # KV heads must split evenly, and a box has at most 8 ranks
    assert el.check_config(cfg(shard_count=4)) == eb.INVALID_REQUEST
    assert el.check_config(cfg(n_head=32, n_head_kv=16, n_vocab=4096, n_embd=4096, n_ff=4096, shard_count=16)) == eb.INVALID_REQUEST
    # the same layouts unsharded are fine
    assert el.check_config(cfg(n_vocab=32002)) == eb.OK
    assert el.check_config(cfg(head_dim=33, rope_dim=32)) == eb.OK
