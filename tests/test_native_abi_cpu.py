"""Layout agreement between the ctypes mirrors and the structures compiled into the kernel library, and the host-only
planning entry points.  None of this launches a kernel, so it runs wherever the library loads (a box without a GPU
included); it catches a field added on one side only before any launch reads a shifted pointer."""
import ctypes as C
import os

import pytest

from smcsd_b200.ops import native as K

_LIB = os.path.join(os.path.dirname(K.__file__), "libsmcsd_b200.so")
pytestmark = pytest.mark.skipif(not os.path.exists(_LIB), reason="kernel library not built")


def test_structure_sizes_match_the_library():
    from smcsd_b200.ops.native_forward import PfParams
    from smcsd_b200.parallel.particle_parallel import PpLocal, PpWorld
    L = K.lib()
    pairs = [(K.SlotArrays, "smc_slot_arrays_size"), (K.CycleIO, "smc_cycle_io_size"), (K.TpLink, "smc_tp_link_size"),
             (K.TpPeers, "smc_tp_peers_size"), (PpWorld, "smc_pp_world_size"), (PpLocal, "smc_pp_local_size"),
             (PfParams, "smc_pf_params_size")]
    for cls, fn in pairs:
        f = getattr(L, fn)
        f.restype = C.c_int
        assert C.sizeof(cls) == f(), f"{cls.__name__} differs from the compiled structure"


def test_split_plans_are_bounded_and_monotone():
    """Key-range split counts of the attention launches: at least one, never more than the cluster limit, and not
    shrinking as the context grows (a plan that shrank would re-key the captured cycle graph back and forth)."""
    prev = 0
    for keys in (64, 256, 1024, 4096, 16384, 65536):
        ks = K.attention_tc_splits(4, 8, keys, 128)
        assert 1 <= ks <= 16 and ks >= prev
        prev = ks
    # more sequences or heads fill the GPU by themselves: fewer splits are planned, never more
    assert K.attention_tc_splits(64, 8, 16384, 128) <= K.attention_tc_splits(1, 8, 16384, 128)
