"""CPU: the bookkeeping of the copy-engine slab chain (gcnasm_b200.peer) -- which slab of which buffer goes where,
which ready word follows it, and the credit that keeps a rank from overwriting a buffer its neighbour still uses.
The three stream primitives are replaced by eager stand-ins over host arrays; `wait` asserts that the value it
waits for is already there, which in this in-order simulation means "its writer was queued before it"."""
import numpy as np
import pytest

from gcnasm_b200.peer import RegionLayout, SlabChain, chain_neighbours


class HostOps:
    """Regions are numpy byte arrays; an address is (rank + 1) << 40 | offset."""

    def __init__(self, world, nbytes):
        self.mem = [np.zeros(nbytes, np.uint8) for _ in range(world)]
        self.log = []

    @staticmethod
    def base(rank):
        return (rank + 1) << 40

    def _at(self, addr):
        return self.mem[(addr >> 40) - 1], addr & ((1 << 40) - 1)

    def copy(self, dst, src, nbytes):
        d, do = self._at(dst)
        s, so = self._at(src)
        d[do:do + nbytes] = s[so:so + nbytes]
        self.log.append(("copy", dst >> 40, src >> 40, nbytes))

    def write(self, addr, value):
        m, o = self._at(addr)
        m[o:o + 4] = np.array([value], np.int32).view(np.uint8)

    def wait(self, addr, value):
        m, o = self._at(addr)
        have = int(m[o:o + 4].view(np.int32)[0])
        if have < value:
            raise AssertionError(f"wait for {value} at rank {(addr >> 40) - 1} offset {o}: the word holds {have}")


def _chains(world, root, lay, ops):
    out = []
    for r in range(world):
        down, up = chain_neighbours(r, world, root)
        out.append(SlabChain(lay, ops, ops.base(r), None if down is None else ops.base(down),
                             None if up is None else ops.base(up), r == root))
    return out


def test_chain_neighbours():
    assert chain_neighbours(0, 4, 0) == (1, None)
    assert chain_neighbours(3, 4, 0) == (None, 2)
    assert chain_neighbours(2, 4, 0) == (3, 1)
    assert chain_neighbours(1, 4, 2) == (None, 0)          # chain 2, 3, 0, 1
    assert chain_neighbours(2, 4, 2) == (3, None)
    assert chain_neighbours(0, 1, 0) == (None, None)


def test_region_layout():
    lay = RegionLayout(slabs=8, bytes_per_slab=17301504, nbuf=2)
    assert lay.act_bytes == 2 * 8 * 17301504 and lay.ready_off % 256 == 0 and lay.ready_off >= lay.act_bytes
    assert lay.credit_off >= lay.ready_off + 4 * 16 and lay.scratch_off > lay.credit_off and lay.total_bytes > lay.scratch_off + 64
    assert lay.slab(1, 3) == (8 + 3) * 17301504 and lay.ready(1, 3) == lay.ready_off + 4 * 11


@pytest.mark.parametrize("world,root", [(2, 0), (4, 0), (8, 0), (4, 2)])
def test_slabs_reach_every_rank_in_order(world, root):
    lay = RegionLayout(slabs=3, bytes_per_slab=64, nbuf=2)
    ops = HostOps(world, lay.total_bytes)
    chains = _chains(world, root, lay, ops)
    order = [(root + i) % world for i in range(world)]
    rng = np.random.default_rng(1)
    for step in range(7):                                   # the two buffers are reused three times
        buf, epoch = step % 2, step + 1
        payload = rng.integers(0, 256, 3 * 64, dtype=np.uint8)
        ops.mem[root][lay.slab(buf, 0):lay.slab(buf, 0) + 3 * 64] = payload        # the root fills its slabs
        touched = []
        for r in order:
            chains[r].forward(step, (lambda s: touched.append(s)) if r == root else None)
        assert touched == [0, 1, 2]
        for r in range(world):
            region = ops.mem[r]
            assert np.array_equal(region[lay.slab(buf, 0):lay.slab(buf, 0) + 3 * 64], payload), (step, r)
            words = region[lay.ready(buf, 0):lay.ready(buf, 0) + 12].view(np.int32)
            assert words.tolist() == [epoch] * 3                                    # what the GEMM of this step waits for
        for r in order:                                     # every rank's GEMM and forwarding of this step are done
            chains[r].credit(step)
        for r in order[:-1]:
            down = chain_neighbours(r, world, root)[0]
            assert int(ops.mem[r][lay.credit_off:lay.credit_off + 4].view(np.int32)[0]) == epoch, (r, down)
    # every data copy is followed by the 4-byte copy of its ready word, to the same neighbour
    copies = [c for c in ops.log if c[0] == "copy"]
    data = [c for c in copies if c[3] == 64]
    flags = [c for c in copies if c[3] == 4]
    assert len(data) == 7 * 3 * (world - 1)
    assert len(flags) == 7 * 3 * (world - 1) + 7 * (world - 1)                     # ready words + credits


def test_a_buffer_is_not_overwritten_before_the_neighbour_is_done():
    """Without the neighbour's credit the third step (first reuse of buffer 0) must not be pushed."""
    lay = RegionLayout(slabs=2, bytes_per_slab=32, nbuf=2)
    ops = HostOps(2, lay.total_bytes)
    chains = _chains(2, 0, lay, ops)
    for step in range(2):
        for r in (0, 1):
            chains[r].forward(step)
    chains[1].credit(0)                                     # rank 1 is done with step 0 only
    chains[0].forward(2)                                    # buffer 0 again: allowed
    with pytest.raises(AssertionError, match="wait for 2"):
        chains[0].forward(3)                                # buffer 1 still holds step 1, which rank 1 has not released
    chains[1].credit(1)
    chains[0].forward(3)


def test_a_rank_forwards_only_what_has_arrived():
    lay = RegionLayout(slabs=2, bytes_per_slab=32, nbuf=2)
    ops = HostOps(3, lay.total_bytes)
    chains = _chains(3, 0, lay, ops)
    with pytest.raises(AssertionError, match="wait for 1"):
        chains[1].forward(0)                                # the root has not pushed anything yet
    chains[0].forward(0)
    chains[1].forward(0)
    chains[2].forward(0)
