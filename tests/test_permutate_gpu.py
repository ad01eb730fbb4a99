"""GPU parity of the general permutation (rank <= 6, `ijk->kij` grammar of
expression_parsing.zig:205-255) against the CPU oracle: bit-exact for alpha = 0."""
import ctypes as C
import itertools

import numpy as np
import pytest

from util import TOL_EW, assert_close, dev, host, narrow, rng_normal, run, wide

pytestmark = pytest.mark.gpu

DTYPES = ["r16", "r32", "r64"]


def len_array(values):
    return (C.c_ulong * len(values))(*[int(v) for v in values])


def out_shape(shape, perm):
    o = [0] * len(shape)
    for i, q in enumerate(perm):
        o[q] = shape[i]
    return tuple(o)


# shapes exercising: odd extents (scalar paths), 16-byte friendly extents (vector paths), size-1 dimensions,
# merges of neighbouring dimensions, tiles cut at both edges, long rows cut into pieces, kept rows of 4 / 8 bytes
# (moved as wider elements)
CASES = [((3, 4, 5), None), ((2, 1, 7, 3), None), ((8, 16, 24), None), ((5, 130, 66), None), ((2, 3, 4, 5, 6), "some"),
         ((2, 3, 2, 3, 2, 3), "some"), ((4, 8, 8, 8, 8, 16), "some"), ((1, 1, 1), None), ((7,), None), ((3, 70000), None),
         ((2, 300, 8), None), ((33, 65, 2), None), ((17, 40, 4), None), ((3, 5, 7, 2), None), ((8, 100, 3, 16), None), ((6, 9, 200), None)]


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("case", CASES, ids=[str(c[0]) for c in CASES])
def test_every_permutation_is_bit_exact(mp, stream, orc, sfx, case):
    shape, pick = case
    perms = list(itertools.permutations(range(len(shape))))
    if pick == "some":
        perms = perms[:: max(1, len(perms) // 16)] + [perms[-1]]
    x = rng_normal(1, shape, sfx)
    xd = dev(x)
    for perm in perms:
        d = dev(np.full(out_shape(shape, perm), np.nan, x.dtype))   # alpha = 0 must not read the fresh output
        run(mp, stream, "permutate", sfx, xd, d, 0.0, len_array(shape), len_array(perm), len(shape))
        ref = narrow(orc.permutate(wide(x), perm), sfx)
        assert np.array_equal(host(d), ref), (shape, perm)


@pytest.mark.parametrize("sfx", DTYPES)
@pytest.mark.parametrize("case", [((3, 4, 5), (1, 2, 0)), ((8, 16, 24), (2, 0, 1)), ((6, 40, 8), (1, 0, 2)), ((37, 53), (1, 0))])
def test_blend_into_the_destination(mp, stream, orc, sfx, case):
    shape, perm = case
    x = rng_normal(2, shape, sfx)
    d0 = rng_normal(3, out_shape(shape, perm), sfx)
    d = dev(d0)
    run(mp, stream, "permutate", sfx, dev(x), d, 0.5, len_array(shape), len_array(perm), len(shape))
    ref = orc.permutate(wide(x), perm, wide(d0).copy(), 0.5)
    assert_close(host(d), narrow(ref, sfx), TOL_EW[sfx], f"permutate alpha=0.5 {shape} {perm}")


@pytest.mark.parametrize("sfx", ["r16", "r32"])
def test_round_trip_at_full_size(mp, stream, sfx):
    # [batch, len, heads, headdim] <-> [batch, heads, len, headdim] and a full reversal, 2^26 elements:
    # permute followed by the inverse permutation restores every bit
    import torch
    shape = (8, 2048, 32, 128)
    x = torch.randn(shape, device="cuda", dtype=torch.float32).to({"r16": torch.float16, "r32": torch.float32}[sfx])
    for perm in [(0, 2, 1, 3), (3, 2, 1, 0), (1, 2, 3, 0)]:
        inv = [0] * 4
        for i, q in enumerate(perm):
            inv[q] = i
        mid_shape = out_shape(shape, perm)
        mid = torch.empty(mid_shape, device="cuda", dtype=x.dtype)
        back = torch.empty_like(x)
        run(mp, stream, "permutate", sfx, x, mid, 0.0, len_array(shape), len_array(perm), 4)
        assert torch.equal(mid, x.permute(*inv).contiguous())
        run(mp, stream, "permutate", sfx, mid, back, 0.0, len_array(mid_shape), len_array(inv), 4)
        assert torch.equal(back, x)


def test_rank2_instance_equals_permutate_ij_ji(mp, stream):
    x = rng_normal(4, (129, 1000), "r32")
    a = dev(np.zeros((1000, 129), np.float32)); b = dev(np.zeros((1000, 129), np.float32))
    run(mp, stream, "permutate_ij_ji", "r32", dev(x), a, 0.0, 129, 1000)
    run(mp, stream, "permutate", "r32", dev(x), b, 0.0, len_array((129, 1000)), len_array((1, 0)), 2)
    assert np.array_equal(host(a), host(b))
