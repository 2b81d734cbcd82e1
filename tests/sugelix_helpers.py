"""Configurations of the Sugelix tests (small sizes of their own, chosen to reach every kernel route).  Model folders,
trace sessions and the error measure are shared with tests/rimidra_helpers.py."""
from oracle import sugelix_oracle as S


def config_mixed():
    """All three mixers, the middle two looped twice, a pair table, an embedding multiplier, grouped heads 4 : 2 and
    2 : 1, a rotation of half the head, windows shorter than the prompts, experts with a shared one."""
    moe = S.moe_mlp(experts=4, top=2, ff=24, limit=1.5, shared_ff=16, shared_limit=0.75)
    return S.make_config([
        S.attention_spec(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, rot_dims=8, base=1000.0, softcap=4.0, mlp=moe),
        S.latent_spec(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=32, scale=0.2, window=12, mlp=moe),
        S.difference_spec(heads=2, kv_heads=1, dim=16, vdim=32, scale=0.25, rot_dims=16, window=9, diff=0.3, base=500.0,
                          factor=2.0, mlp=moe),
        S.attention_spec(heads=2, kv_heads=2, dim=16, vdim=8, scale=0.25, rot_dims=16, base=100.0, softcap=30.0, mlp=None),
    ], width=64, vocab=96, embed_scale=4.0, bigram=(61, 31, 5), loop=(1, 3, 2))


def config_ones():
    """What a usual model makes > 1 is 1 or absent here: no pair table, no loop, multiplier 1, one head, one key/value
    head, windows of one token, top 1 of two experts, no shared expert, no cap, no rotation in one layer, a layer
    without feed-forward; sizes off the multiples of 8 (CUDA-core GEMMs even in 16 bits)."""
    one = S.moe_mlp(experts=2, top=1, ff=10, limit=7.0)
    return S.make_config([
        S.attention_spec(heads=1, kv_heads=1, dim=10, vdim=6, scale=1.0, rot_dims=0, mlp=one),
        S.difference_spec(heads=1, kv_heads=1, dim=6, vdim=10, scale=0.5, rot_dims=2, window=1, diff=0.8, mlp=None),
        S.latent_spec(heads=1, dim=6, rot_dim=2, vdim=12, q_rank=5, kv_rank=7, scale=0.4, window=1, mlp=one),
        S.latent_spec(heads=3, dim=4, rot_dim=6, vdim=4, q_rank=9, kv_rank=11, scale=0.3, window=3, mlp=None),
    ], width=36, vocab=50, eps=1e-5)


def config_wide():
    """Shapes that the tensor-core GEMMs and attention kernels tile: key 64 / value 64, two maps of key 64 over values
    of 128, a latent row of 64 + 64 read as keys of 128 and values of 64; grouped heads 8 : 2; every layer inside a
    loop of three passes; five experts, three chosen; a window that crosses the cache's run length."""
    moe = S.moe_mlp(experts=5, top=3, ff=64, limit=2.0, shared_ff=128, shared_limit=1.0)
    return S.make_config([
        S.attention_spec(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.12, rot_dims=32, base=3e5, softcap=15.0, mlp=moe),
        S.difference_spec(heads=4, kv_heads=2, dim=64, vdim=128, scale=0.125, rot_dims=64, window=140, diff=0.6,
                          base=2e5, factor=8.0, mlp=moe),
        S.latent_spec(heads=4, dim=32, rot_dim=64, vdim=64, q_rank=48, kv_rank=64, scale=0.1, window=40, mlp=moe),
    ], width=256, vocab=264, embed_scale=8.0, bigram=(127, 97, 3), loop=(0, 3, 3))


def config_far():
    """Sharp attention (weights with a gain that makes every query look at one key, wherever it is) and windows longer
    than the prompts: a token hundreds back, or the one at a window's edge, decides the logits."""
    return S.make_config([
        S.attention_spec(heads=2, kv_heads=1, dim=16, vdim=16, scale=1.0, rot_dims=4, base=50.0, softcap=50.0, mlp=None),
        S.difference_spec(heads=2, kv_heads=2, dim=8, vdim=16, scale=1.5, rot_dims=8, window=500, diff=0.2, mlp=None),
        S.latent_spec(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=16, kv_rank=16, scale=1.5, window=7,
                      mlp=S.moe_mlp(experts=3, top=2, ff=16, limit=1.0)),
    ], width=32, vocab=64, bigram=(13, 7, 11))


def config_uneven():
    """Sizes in whole 16-byte vectors that no attention tile and few GEMM tiles fit: three query heads per key head,
    values wider than keys and narrower, six experts of which three are chosen, a loop that starts at the first layer
    and leaves the last one out, a window of exactly the cache's run length."""
    moe = S.moe_mlp(experts=6, top=3, ff=40, limit=3.0, shared_ff=72, shared_limit=0.5)
    return S.make_config([
        S.latent_spec(heads=5, dim=24, rot_dim=16, vdim=40, q_rank=72, kv_rank=48, scale=0.15, window=128, base=3000.0,
                      mlp=moe),
        S.attention_spec(heads=6, kv_heads=2, dim=32, vdim=80, scale=0.18, rot_dims=24, base=7e4, softcap=8.0, mlp=moe),
        S.difference_spec(heads=6, kv_heads=3, dim=40, vdim=16, scale=0.16, rot_dims=40, window=50, diff=0.65, base=9e3,
                          factor=3.0, mlp=moe),
    ], width=192, vocab=300, embed_scale=2.5, bigram=(211, 5, 9), loop=(0, 2, 2))


CONFIGS = {"mixed": config_mixed, "ones": config_ones, "wide": config_wide, "far": config_far, "uneven": config_uneven}
SEEDS = {"mixed": 5, "ones": 2, "wide": 8, "far": 4, "uneven": 6}
