"""The work partition of the SSD chunk walk (one CTA per SM slot, every CTA the same number of chunks, a sequence cut
between two CTAs hands its state over once) through the host-side copy of the function the kernels use.  No GPU."""
import ctypes as C

import pytest


@pytest.fixture(scope="module")
def partition():
    import metaphor_b200 as mp
    fn = mp.lib().mpSsdWalkPartition

    def segments(cta, ncta, nseq, nc):
        out, idx, buf = [], 0, (C.c_int * 5)()
        while fn(cta, ncta, nseq, nc, idx, buf):
            out.append(tuple(buf))
            idx += 1
            assert idx < 10000
        return out
    return segments


# (sequences, chunks per sequence, CTAs): the language model's forward and one of its reverse walks, the scan benchmark's
# forward and reverse walk, one CTA per sequence, a single CTA, a range that ends exactly on sequence boundaries
CASES = [(192, 16, 148), (192, 16, 74), (256, 64, 148), (256, 64, 74), (12, 5, 12), (7, 3, 1), (300, 4, 100), (149, 2, 148), (160, 3, 148)]


@pytest.mark.parametrize("nseq,nc,ncta", CASES)
def test_every_chunk_is_walked_once_and_states_are_handed_forward(partition, nseq, nc, ncta):
    walked = {}
    carried_out, carried_in = {}, {}
    total = nseq * nc
    for cta in range(ncta):
        segs = partition(cta, ncta, nseq, nc)
        assert segs, "every CTA has work"
        count = sum(n for _, _, n, _, _ in segs)
        assert total // ncta <= count <= total // ncta + 1, "equal shares"
        assert count >= nc, "a range is at least one sequence long"
        for i, (seq, p0, n, cin, cout) in enumerate(segs):
            assert 0 <= seq < nseq and n >= 1 and 0 <= p0 and p0 + n <= nc
            assert (cin == 1) == (p0 > 0), "a state is carried in exactly when the segment starts inside a sequence"
            assert (cout == 1) == (p0 + n < nc), "... and out when it ends inside one"
            assert not (cin and cout), "a segment inside one sequence would chain CTAs"
            if cout:
                assert i == 0, "the part that hands a state on is walked first"
                carried_out[seq] = cta
            if cin:
                assert i == len(segs) - 1, "the part that receives a state is walked last"
                carried_in[seq] = cta
            for p in range(p0, p0 + n):
                assert (seq, p) not in walked
                walked[(seq, p)] = cta
    assert len(walked) == total
    assert carried_in.keys() == carried_out.keys()
    for seq, cta in carried_in.items():
        assert carried_out[seq] == cta - 1, "the state comes from the neighbouring CTA, which produced it in its first segment"


def test_arguments_outside_the_contract_yield_no_segment(partition):
    assert partition(0, 8, 4, 16) == []      # more CTAs than sequences
    assert partition(5, 4, 8, 16) == []      # CTA index out of range
