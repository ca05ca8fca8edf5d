"""Host <-> device state transfers beyond the one-block byte upload: several blocks per call, bit-packed uploads (the
mirror of the bit-packed state stream) and chain-range downloads.  All must land the same bytes in the device state."""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chains", [1, 16, 37, 70, 256, 1030])
def test_packed_and_many_uploads_equal_byte_upload(T, chains):
    desc, info = M.ising_random_graph(T, 150, 6, 3)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    nb = len(desc["free"])
    init = M.random_states(desc, chains, 11)
    ref = T.ChainState(prog, chains)
    for b, a in enumerate(init):
        ref.upload(b, a)
    many, packed = T.ChainState(prog, chains), T.ChainState(prog, chains)
    many.upload_many(list(range(nb)), init)
    packed.upload_packed(list(range(nb)), [T.pack_chains(a) for a in init])
    for b in range(nb):
        want = ref.download(b, np.uint8)
        assert np.array_equal(want, init[b])
        assert np.array_equal(many.download(b, np.uint8), want)
        assert np.array_equal(packed.download(b, np.uint8), want)
    # the padding chains of a packed upload are zero, so the next sweep sees the same state: same bits afterwards
    ref.run_blocks(3, 2)
    packed.run_blocks(3, 2)
    for b in range(nb):
        assert np.array_equal(ref.download(b, np.uint8), packed.download(b, np.uint8))
    # round trip through the bit-packed state stream
    bits = packed.sample_states_packed(9, 0, 1, 1, list(range(nb)))[0]
    again = T.ChainState(prog, chains)
    rows = np.cumsum([0] + [len(f[0]) for f in desc["free"]])
    again.upload_packed(list(range(nb)), [bits[rows[b]:rows[b + 1]] for b in range(nb)])
    for b in range(nb):
        assert np.array_equal(again.download(b, np.uint8), packed.download(b, np.uint8))


def test_chain_range_download(T):
    desc, info = M.ising_random_graph(T, 90, 6, 5)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    chains = 200
    st = T.ChainState(prog, chains)
    init = M.random_states(desc, chains, 2)
    for b, a in enumerate(init):
        st.upload(b, a)
    for begin, cnt in [(0, 200), (0, 1), (199, 1), (16, 33), (37, 100)]:
        assert np.array_equal(st.download_chains(1, begin, cnt), init[1][begin:begin + cnt])
    with pytest.raises(T.ThrmlError, match="chain range"):
        st.download_chains(0, 190, 20)


def test_packed_upload_rejects_categorical_blocks(T):
    desc, info = M.potts_lattice(T, 4, 3, 1)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    st = T.ChainState(prog, 32)
    with pytest.raises(T.ThrmlError, match="spin blocks"):
        st.upload_packed([0], [np.zeros((8, 1), np.uint32)])
