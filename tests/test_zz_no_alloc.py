"""The allocation-free upload entry point (thrml_state_upload_u8_static), called through the C ABI.

It exists for hosts that cannot call cudaMalloc while they run (GPU memory already committed elsewhere, or no tolerance
for the device-wide synchronisation an allocation implies).  Its result must be byte-identical to the ordinary upload's,
on repeated calls that reuse the library's fixed staging array, and oversized blocks must be refused with a clear error.
This file is collected last so that a run stopping at the first failure has already executed every other test.
"""
import numpy as np
import pytest

import models as M

pytestmark = pytest.mark.gpu


def test_static_upload_matches_ordinary_upload_twice(T):
    desc, _ = M.ising_random_graph(T, 400, 8, 71)
    prog = T.Program(M.fill(T.Builder(desc["kinds"]), desc))
    n_blocks = len(desc["free"])
    for chains in (37, 256):  # ragged and aligned chain counts; the second pass reuses the array after a larger first one
        ref, sta = T.ChainState(prog, chains), T.ChainState(prog, chains)
        for call in range(2):  # two calls in a row on the same handles
            init = M.random_states(desc, chains, 100 + call)
            for b, a in enumerate(init):
                ref.upload(b, a)
                sta.upload_static(b, a)
            for b in range(n_blocks):
                want, got = ref.download(b, np.uint8), sta.download(b, np.uint8)
                assert np.array_equal(got, init[b]) and np.array_equal(got, want)
            ref.run_blocks(9 + call, 2)
            sta.run_blocks(9 + call, 2)
            for b in range(n_blocks):
                assert np.array_equal(ref.download(b, np.uint8), sta.download(b, np.uint8))


def test_static_upload_rejects_blocks_beyond_its_scratch(T):
    n = 5000
    bld = T.Builder(np.zeros(n, np.int32))
    bld.add_free_block(np.arange(n))
    bld.compile()
    st = T.ChainState(T.Program(bld), 1024)  # 5000 x 1024 bytes > 4 MiB
    with pytest.raises(T.ThrmlError, match="exceeds the static scratch"):
        st.upload_static(0, np.zeros((1024, n), np.uint8))
    st.upload(0, np.ones((1024, n), np.uint8))  # the ordinary entry point still takes it
    assert st.download(0, np.uint8).all()
