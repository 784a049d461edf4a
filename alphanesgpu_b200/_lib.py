"""ctypes binding of libstafb.so (the C ABI declared in include/stafb.h).

There is no fallback: if the shared library is missing the import of any op raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libstafb.so")

OK = 0
STATUS_NAMES = {1: "RADIAL_OVERFLOW", 2: "ANGULAR_OVERFLOW", 3: "CELL_OVERFLOW", 4: "BAD_BOX", 5: "INVALID",
                6: "CUDA", 7: "CAPACITY", 8: "NONFINITE", 9: "PEER_TIMEOUT", 10: "STAGE_TIMEOUT"}


class StafbError(RuntimeError):
    def __init__(self, status, where=""):
        self.status = status
        msg = lib().stafb_strerror(status).decode()
        if status == 6:
            msg += ": " + lib().stafb_last_cuda_error().decode()
        super().__init__("%s: status %d (%s)" % (where or "stafb", status, msg))


_LIB = None
_vp, _i, _d = C.c_void_p, C.c_int, C.c_double

_SIGS = {
    "stafb_create": [C.POINTER(_vp), _i, _d, _d, _d, _i, _i, _i, _i],
    "stafb_destroy": [_vp],
    "stafb_status": [_vp, _vp],
    "stafb_core_coefficients": [_vp, _vp],
    "stafb_last_launch_count": [_vp],
    "stafb_compute_descriptors_light": [_vp, _vp, _vp, _vp, _i, _i] + [_vp] * 9,
    "stafb_compute_sort_proj": [_vp, _vp] + [_vp] * 5 + [_i] * 4 + [_vp],
    "stafb_compute_sort_proj3body": [_vp, _vp] + [_vp] * 8 + [_i] * 4 + [_vp],
    "stafb_compute_force_radial": [_vp, _vp] + [_vp] * 9 + [_i] * 5 + [_vp],
    "stafb_compute_force_tripl": [_vp, _vp] + [_vp] * 13 + [_i] * 5 + [_vp],
    "stafb_compute_two_body_par_grad": [_vp, _vp] + [_vp] * 6 + [_i] * 4 + [_vp] * 2,
    "stafb_compute_sort_proj3body_grad": [_vp, _vp] + [_vp] * 9 + [_i] * 4 + [_vp] * 2,
    "stafb_compute_force_radial_grad": [_vp, _vp] + [_vp] * 10 + [_i] * 5 + [_vp] * 3,
    "stafb_compute_force_tripl_grad": [_vp, _vp] + [_vp] * 14 + [_i] * 5 + [_vp] * 3,
    "stafb_compute_force_radial_virial": [_vp, _vp] + [_vp] * 11 + [_i] * 5 + [_vp] * 2,
    "stafb_compute_force_tripl_virial": [_vp, _vp] + [_vp] * 15 + [_i] * 5 + [_vp] * 2,
    "stafb_compute_force_radial_virial_grad": [_vp, _vp] + [_vp] * 13 + [_i] * 5 + [_vp] * 3,
    "stafb_compute_force_tripl_virial_grad": [_vp, _vp] + [_vp] * 17 + [_i] * 5 + [_vp] * 3,
    "stafb_init_force_radial": [_i], "stafb_init_force_tripl": [_i],
    "stafb_init_grad_force_radial": [_i], "stafb_init_grad_force_tripl": [_i],
    "stafb_model_create": [_vp, _vp, C.POINTER(_vp)],
    "stafb_model_destroy": [_vp],
    "stafb_model_n_params": [_vp],
    "stafb_model_n_emb": [_vp],
    "stafb_model_offsets": [_vp, _i, _vp],
    "stafb_model_mlp_config": [_vp, _vp],
    "stafb_model_mlp_mma_config": [_vp, _vp],
    "stafb_energy_force": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp],
    "stafb_energy_force_virial": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp],
    "stafb_energy_force_domain": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "stafb_model_set_counts": [_vp, _vp],
    "stafb_train_step": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _i, _vp, _vp, _vp, _vp],
    "stafb_train_step_virial": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _d, _i, _vp, _vp,
                                _vp, _vp, _vp],
    "stafb_descriptors_prefetch": [_vp, _vp, _vp, _vp, _vp, _i, _i],
    "stafb_train_step_prefetched": [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _i, _vp, _vp, _vp,
                                    _vp],
    "stafb_peer_create": [_vp, _i, _i, _i, _vp],
    "stafb_peer_handle": [_vp, _vp],
    "stafb_peer_connect": [_vp, _vp],
    "stafb_peer_status": [_vp],
    "stafb_peer_connect_local": [_vp, _vp],
    "stafb_peer_grad": [_vp, _i],
    "stafb_peer_set_wait_ms": [_vp, C.c_longlong],
    "stafb_peer_destroy": [_vp],
    "stafb_halo_create": [_vp, _i, _i, _i, _i, _vp],
    "stafb_halo_handle": [_vp, _vp],
    "stafb_halo_connect": [_vp, _vp],
    "stafb_halo_connect_local": [_vp, _vp],
    "stafb_halo_positions": [_vp],
    "stafb_halo_forces": [_vp],
    "stafb_halo_set_wait_ms": [_vp, C.c_longlong],
    "stafb_halo_set_plan": [_vp, _vp, _i, _i, _i, _vp, _i, _i, _vp, _i, _i],
    "stafb_halo_plan_select": [_vp, _vp, _i, _vp, _i, _d, _d],
    "stafb_halo_plan_layout": [_vp, _vp, _vp],
    "stafb_halo_plan_done": [_vp, _vp],
    "stafb_halo_plan_finish": [_vp, _vp, _vp],
    "stafb_halo_push_positions": [_vp, _vp],
    "stafb_halo_wait_positions": [_vp, _vp],
    "stafb_halo_return_forces": [_vp, _vp, _vp, _vp],
    "stafb_halo_collect": [_vp, _vp, _vp, _vp],
    "stafb_halo_status": [_vp],
    "stafb_halo_destroy": [_vp],
    "stafb_allreduce_adam": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _d, _d, _d, _d, _vp],
    "stafb_allreduce_adam_phase": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _d, _d, _d, _d, _vp, _i],
    "stafb_train_step_host": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _i, _vp, _vp],
    "stafb_train_step_host_begin": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _i, _vp, _i],
    "stafb_train_step_host_end": [_vp, _vp, _i, _vp],
    "stafb_train_step_virial_host_begin": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _d, _d, _d, _d, _d, _i,
                                           _vp, _i],
    "stafb_train_step_virial_host_end": [_vp, _vp, _i, _vp],
    "stafb_adam_step_dev": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _d, _d, _d, _d, _vp, _d],
    "stafb_measure_fma_peak": [_i, _vp, _vp],
    "stafb_set_phase_timing": [_vp, _i],
    "stafb_get_phase_times": [_vp, _vp, _i],
    "stafb_adam_step": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _d, _d, _d, _d, _i, _d],
}


def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "alphanesgpu_b200: %s is missing - build it with `python -m alphanesgpu_b200.build` "
                "(needs nvcc); there is no CPU fallback" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        L.stafb_strerror.restype = C.c_char_p
        L.stafb_strerror.argtypes = [_i]
        L.stafb_last_cuda_error.restype = C.c_char_p
        for name, sig in _SIGS.items():
            fn = getattr(L, name, None)
            if fn is None:
                continue
            fn.argtypes = sig
            fn.restype = None if name in ("stafb_destroy", "stafb_model_destroy", "stafb_core_coefficients",
                                          "stafb_model_offsets", "stafb_peer_destroy", "stafb_model_mlp_config",
                                          "stafb_model_mlp_mma_config",
                                          "stafb_halo_destroy") else _i
            if name in ("stafb_peer_grad", "stafb_halo_positions", "stafb_halo_forces"):
                fn.restype = C.c_void_p
        _LIB = L
    return _LIB


def check(status, where=""):
    if status != OK:
        raise StafbError(status, where)
