"""Configurations of the Matepel tests (small sizes of their own, chosen to reach every kernel route).  Model folders,
trace sessions and the error measure are shared with tests/rimidra_helpers.py."""
from oracle import matepel_oracle as M


def config_mixed():
    """Both mixers with and without a feed-forward, two streams, grouped heads 4 : 2, a rotation of half the head
    with rescaled frequencies, branch scales and a residual multiplier off 1."""
    return M.make_config([
        M.lightning_spec(heads=2, dim=16, vdim=32, mlp=M.dense_mlp(48, limit=1.0)),
        M.parallel_spec(heads=4, kv_heads=2, dim=16, scale=0.3, rot_dims=8, base=10000.0, scaling=(4.0, 64, 8.0, 1.0),
                        r_heads=2, r_dim=16, r_vdim=32, gate_cap=12.0, left_scale=0.75, right_scale=1.1,
                        mlp=M.dense_mlp(40, limit=2.0)),
        M.lightning_spec(heads=2, dim=16, vdim=32, decay=[0.7, 0.98], mlp=None),
        M.parallel_spec(heads=2, kv_heads=2, dim=16, scale=0.25, rot_dims=16, base=500.0, scaling=None,
                        r_heads=1, r_dim=24, r_vdim=40, gate_cap=6.0, left_scale=1.2, right_scale=0.5, mlp=None),
    ], width=64, vocab=96, streams=2, residual_mult=0.6)


def config_ones():
    """What a usual model makes > 1 is 1 here: one stream (with its coefficients), one head everywhere, one key/value
    head, multiplier and scales 1, no rotation in one layer and a whole-head rotation in the other; sizes off the
    multiples of 8 (CUDA-core GEMMs even in 16 bits)."""
    return M.make_config([
        M.parallel_spec(heads=1, kv_heads=1, dim=10, scale=1.0, rot_dims=0, r_heads=1, r_dim=12, r_vdim=6, gate_cap=9.0,
                        mlp=M.dense_mlp(20, limit=7.0)),
        M.lightning_spec(heads=1, dim=12, vdim=10, decay=[1.0], mlp=None),
        M.parallel_spec(heads=1, kv_heads=1, dim=12, scale=0.5, rot_dims=12, base=100.0, r_heads=1, r_dim=10, r_vdim=36,
                        gate_cap=1.0, mlp=None),
    ], width=36, vocab=50, streams=1, residual_mult=1.0, eps=1e-5)


def config_wide():
    """Shapes that the tensor-core GEMMs and attention tile: key size 64 and 128 in the recurrences, value size twice
    and half the key size, grouped heads 8 : 2 and 6 : 1, four streams, three query heads per key head off the
    powers of two."""
    return M.make_config([
        M.lightning_spec(heads=4, dim=64, vdim=128, mlp=M.dense_mlp(192, limit=1.5)),
        M.parallel_spec(heads=8, kv_heads=2, dim=64, scale=0.12, rot_dims=32, base=3e5, scaling=(8.0, 128, 32.0, 1.0),
                        r_heads=2, r_dim=64, r_vdim=128, gate_cap=18.0, left_scale=0.9, right_scale=0.7,
                        mlp=M.dense_mlp(128, limit=1.0)),
        M.parallel_spec(heads=6, kv_heads=1, dim=32, scale=0.2, rot_dims=16, base=1e4, scaling=(2.0, 32, 4.0, 2.0),
                        r_heads=4, r_dim=128, r_vdim=32, gate_cap=10.0, mlp=None),
        M.lightning_spec(heads=2, dim=128, vdim=64, decay=[0.95, 0.9999], mlp=None),
    ], width=256, vocab=264, streams=4, residual_mult=0.5)


def config_far():
    """No stream key at all (one plain residual), sharp attention (a scale that makes every query look at one key,
    wherever it is) and memories that hardly forget: a token hundreds back decides the logits."""
    return M.make_config([
        M.parallel_spec(heads=2, kv_heads=1, dim=16, scale=3.0, rot_dims=4, base=50.0, r_heads=2, r_dim=8, r_vdim=16,
                        gate_cap=14.0, mlp=None),
        M.lightning_spec(heads=2, dim=8, vdim=16, decay=[1.0, 0.9995], mlp=M.dense_mlp(32, limit=1.0)),
    ], width=32, vocab=64, streams=None, residual_mult=0.8)


CONFIGS = {"mixed": config_mixed, "ones": config_ones, "wide": config_wide, "far": config_far}
SEEDS = {"mixed": 4, "ones": 1, "wide": 7, "far": 3}
