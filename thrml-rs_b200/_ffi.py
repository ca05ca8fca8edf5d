"""ctypes declarations for libthrml_b200.so (the C ABI of include/thrml_b200.h).

The library is the only compute path of this package: if it cannot be loaded the import fails, and every device
call fails with the library's own error when no CUDA device is usable.  There is no Python or CPU fallback.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

OK = 0
ERR_NAMES = {-1: "INVALID_ARG", -2: "BAD_COLOURING", -3: "CUDA", -4: "NCCL", -5: "TIMEOUT", -6: "OOM", -7: "UNSUPPORTED"}

# Every symbol the header declares, with argument types.  tests/test_abi.py checks this list against the header.
_P = C.c_void_p
_SIGNATURES = {
    "thrml_last_error": (C.c_char_p, []),
    "thrml_version": (C.c_char_p, []),
    "thrml_rng_split": (C.c_int32, [C.c_uint64, C.c_int64, _P]),
    "thrml_lattice_edges": (C.c_int32, [C.c_int64, C.c_int32, _P, _P, _P, _P]),
    "thrml_greedy_coloring": (C.c_int32, [C.c_int64, C.c_int64, _P, _P, _P]),
    "thrml_builder_create": (C.c_int32, [_P, C.c_int64, _P, C.c_int32, _P]),
    "thrml_builder_destroy": (None, [_P]),
    "thrml_builder_add_free_block": (C.c_int32, [_P, _P, C.c_int64, C.c_int32, C.c_int32]),
    "thrml_builder_add_clamped_block": (C.c_int32, [_P, _P, C.c_int64]),
    "thrml_builder_add_interaction_group": (C.c_int32, [_P, _P, C.c_int64, _P, C.c_int32, C.c_int32, _P, C.c_int32, C.c_int32]),
    "thrml_builder_add_discrete_factor": (C.c_int32, [_P, _P, C.c_int32, _P, C.c_int32, C.c_int64, _P, C.c_int32, C.c_int32, _P]),
    "thrml_builder_add_ising": (C.c_int32, [_P, _P, C.c_int64, _P, _P, C.c_int64, _P, C.c_float]),
    "thrml_builder_compile": (C.c_int32, [_P]),
    "thrml_builder_counts": (C.c_int32, [_P, _P, _P, _P, _P]),
    "thrml_builder_node_location": (C.c_int32, [_P, C.c_int64, _P, _P]),
    "thrml_builder_group_shape": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "thrml_builder_group_data": (C.c_int32, [_P, C.c_int32, _P, _P, _P]),
    "thrml_builder_block_tables": (C.c_int32, [_P, C.c_int32, _P, _P]),
    "thrml_builder_table_shape": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "thrml_builder_table_data": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, _P, _P, _P, _P]),
    "thrml_ctx_create": (C.c_int32, [C.c_int32, _P]),
    "thrml_ctx_destroy": (None, [_P]),
    "thrml_builder_compile_device": (C.c_int32, [_P, _P]),
    "thrml_greedy_coloring_device": (C.c_int32, [_P, C.c_int64, C.c_int64, _P, _P, _P, _P]),
    "thrml_ctx_synchronize": (C.c_int32, [_P]),
    "thrml_ctx_stream": (C.c_void_p, [_P]),
    "thrml_debug_wait_timeout": (C.c_int32, [_P]),
    "thrml_program_update_group": (C.c_int32, [_P, C.c_int32, _P, C.c_int64, C.c_int32, C.c_float]),
    "thrml_estimate_kl_grad": (C.c_int32, [_P, _P, _P, _P, C.c_uint64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float, _P, _P]),
    "thrml_program_set_option": (C.c_int32, [_P, C.c_int32, C.c_double]),
    "thrml_program_get_option": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_debug_pair_tmem_check": (C.c_int32, [_P]),
    "thrml_program_create": (C.c_int32, [_P, _P, _P]),
    "thrml_program_destroy": (None, [_P]),
    "thrml_program_update_weights": (C.c_int32, [_P, C.c_int32, C.c_int32, _P]),
    "thrml_program_block_kernel": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_program_enable_dense": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_ising_energy": (C.c_int32, [_P, C.c_int64, _P, _P, C.c_int64, _P, _P, C.c_float, _P]),
    "thrml_factor_energy": (C.c_int32, [_P, C.c_int64, C.c_int32, C.c_int32, _P, _P, C.c_int32, C.c_int32, _P]),
    "thrml_sample_single_block": (C.c_int32, [_P, C.c_int32, C.c_uint64]),
    "thrml_pair_correlation": (C.c_int32, [_P, C.c_int32, C.c_int32, _P]),
    "thrml_cd1_step": (C.c_int32, [_P, C.c_int32, C.c_int32, _P, C.c_uint64, _P, _P]),
    "thrml_cd1_step_from": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, C.c_uint64, _P, _P]),
    "thrml_cd1_step_comm": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, C.c_uint64, _P, _P, _P]),
    "thrml_state_create": (C.c_int32, [_P, C.c_int64, C.c_int64, _P]),
    "thrml_state_destroy": (None, [_P]),
    "thrml_state_upload_f32": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_state_download_f32": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_state_upload_u8": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_state_download_u8": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_state_download_chains_u8": (C.c_int32, [_P, C.c_int32, C.c_int64, C.c_int64, _P]),
    "thrml_state_upload_u8_static": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_state_upload_u8_many": (C.c_int32, [_P, _P, C.c_int32, _P]),
    "thrml_state_upload_packed": (C.c_int32, [_P, _P, C.c_int32, _P]),
    "thrml_comm_unique_id": (C.c_int32, [_P]),
    "thrml_comm_create": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, _P]),
    "thrml_comm_adopt": (C.c_int32, [_P, _P, _P]),
    "thrml_comm_destroy": (None, [_P]),
    "thrml_comm_info": (C.c_int32, [_P, _P, _P, _P]),
    "thrml_moments_allreduce": (C.c_int32, [_P, _P]),
    "thrml_state_copy_block": (C.c_int32, [_P, _P, C.c_int32]),
    "thrml_hinton_init": (C.c_int32, [_P, _P, C.c_int32, _P, C.c_float, C.c_uint64, _P]),
    "thrml_state_randomize": (C.c_int32, [_P, C.c_uint64]),
    "thrml_sample_blocks": (C.c_int32, [_P, C.c_uint64, _P]),
    "thrml_run_blocks": (C.c_int32, [_P, C.c_uint64, C.c_int64, _P]),
    "thrml_fields_debug": (C.c_int32, [_P, C.c_int32, _P]),
    "thrml_moments_create": (C.c_int32, [_P, C.c_int32, _P, _P, _P, C.c_int32, _P]),
    "thrml_moments_destroy": (None, [_P]),
    "thrml_moments_reset": (C.c_int32, [_P]),
    "thrml_moments_observe": (C.c_int32, [_P, _P]),
    "thrml_moments_read": (C.c_int32, [_P, C.c_int32, _P, _P]),
    "thrml_moments_device_buffer": (C.c_int32, [_P, _P, _P]),
    "thrml_moments_add_observations": (C.c_int32, [_P, C.c_int64]),
    "thrml_moments_fused_info": (C.c_int32, [_P, _P, _P]),
    "thrml_state_launch_counts": (C.c_int32, [_P, _P, _P]),
    "thrml_marginals_create": (C.c_int32, [_P, _P, C.c_int32, C.c_int32, _P]),
    "thrml_sample_states_packed": (C.c_int32, [_P, C.c_uint64, C.c_int64, C.c_int64, C.c_int64, _P, C.c_int32, _P]),
    "thrml_lattice_create": (C.c_int32, [_P, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_int64, C.c_int64, _P]),
    "thrml_lattice_destroy": (None, [_P]),
    "thrml_lattice_randomize": (C.c_int32, [_P, C.c_uint64]),
    "thrml_lattice_upload": (C.c_int32, [_P, _P]),
    "thrml_lattice_download": (C.c_int32, [_P, _P]),
    "thrml_lattice_set_noise": (C.c_int32, [_P, C.c_int32]),
    "thrml_lattice_upload_bits": (C.c_int32, [_P, _P]),
    "thrml_lattice_download_bits": (C.c_int32, [_P, _P]),
    "thrml_lattice_update": (C.c_int32, [_P, C.c_int32, C.c_uint64, C.c_int64, C.c_int64]),
    "thrml_lattice_halo_info": (C.c_int32, [_P, C.c_int32, _P, _P, _P, _P, _P]),
    "thrml_lattice_copy_halo": (C.c_int32, [_P, C.c_int32, _P, C.c_int32, C.c_int32]),
    "thrml_lattice_wrap_halo": (C.c_int32, [_P, C.c_int32]),
    "thrml_lattice_observe": (C.c_int32, [_P, _P]),
    "thrml_lattice_synchronize": (C.c_int32, [_P]),
    "thrml_lattice_run_blocks": (C.c_int32, [_P, C.c_uint64, C.c_int64, _P, C.c_int32]),
    "thrml_lattice_refresh_halos": (C.c_int32, [_P, _P]),
    "thrml_lattice_read_series": (C.c_int32, [_P, _P, _P, C.c_int64, _P]),
    "thrml_lattice_moments": (C.c_int32, [_P, _P, _P, _P]),
    "thrml_lattice_series_reset": (C.c_int32, [_P]),
    "thrml_potts_create": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, C.c_float, C.c_int64, C.c_int64, _P]),
    "thrml_potts_destroy": (None, [_P]),
    "thrml_potts_set_noise": (C.c_int32, [_P, C.c_int32]),
    "thrml_potts_randomize": (C.c_int32, [_P, C.c_uint64]),
    "thrml_potts_upload": (C.c_int32, [_P, _P]),
    "thrml_potts_download": (C.c_int32, [_P, _P]),
    "thrml_potts_update": (C.c_int32, [_P, C.c_int32, C.c_uint64]),
    "thrml_potts_observe_marginals": (C.c_int32, [_P]),
    "thrml_potts_read_marginals": (C.c_int32, [_P, _P, _P]),
    "thrml_potts_reset_marginals": (C.c_int32, [_P]),
    "thrml_potts_synchronize": (C.c_int32, [_P]),
    "thrml_potts_run_blocks": (C.c_int32, [_P, C.c_uint64, C.c_int64]),
    "thrml_potts_sample_with_marginals": (C.c_int32, [_P, C.c_uint64, C.c_int64, C.c_int64, C.c_int64]),
    "thrml_potts_marginals_allreduce": (C.c_int32, [_P, _P]),
    "thrml_sample_with_observation": (C.c_int32, [_P, C.c_uint64, C.c_int64, C.c_int64, C.c_int64, _P, _P, C.c_int32, _P, _P]),
}


class Noise(C.Structure):
    _fields_ = [("u", C.c_void_p), ("len", C.c_int64)]


class ThrmlError(ValueError):
    """A failing C-ABI call; `code` is the THRML_ERR_* status, the message is thrml_last_error()."""

    def __init__(self, code, msg):
        super().__init__(f"[{ERR_NAMES.get(code, code)}] {msg}")
        self.code = code
        self.message = msg


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.OUT
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc); there is no fallback path")
        _lib = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def check(rc):
    if rc != OK:
        raise ThrmlError(rc, lib().thrml_last_error().decode())


def ptr(a):
    """Pointer to a C-contiguous numpy array (or None)."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def make_noise(u):
    if u is None:
        return None, None
    u = f32(u).ravel()
    nz = Noise(u.ctypes.data, u.size)
    return nz, u  # keep `u` alive while the struct is in use
