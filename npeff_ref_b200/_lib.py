"""ctypes binding of ``libdnpeff.so`` (the C ABI declared in include/dnpeff.h)."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

OK = 0
N_TIMERS = 6
TIMER_NAMES = ("spmm_ah", "spmm_wa", "gram", "mu_update", "allreduce", "loss")


class DnpeffError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("dnpeff error %d: %s" % (code, message))
        self.code = code


class Params(C.Structure):
    _fields_ = [("rank", C.c_int32), ("eps", C.c_float), ("seed", C.c_uint64),
                ("init_scale", C.c_float), ("shard_index", C.c_int32), ("n_shards", C.c_int32),
                ("shard_mode", C.c_int32)]


def lib_path():
    return os.path.join(_HERE, "libdnpeff.so")


# name -> (restype, argtypes); every symbol include/dnpeff.h declares.
_P = C.c_void_p
_I64 = C.c_int64
_I32 = C.c_int32
SIGNATURES = {
    "dnpeff_last_error": (C.c_char_p, []),
    "dnpeff_abi_version": (C.c_int, []),
    "dnpeff_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "dnpeff_create": (C.c_int, [C.POINTER(Params), C.c_int, _P, C.POINTER(_P)]),
    "dnpeff_destroy": (C.c_int, [_P]),
    "dnpeff_set_option": (C.c_int, [_P, C.c_char_p, _I64]),
    "dnpeff_set_csr": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _I32]),
    "dnpeff_row_slice": (C.c_int, [_I64, _I32, _I32, C.POINTER(_I64), C.POINTER(_I64)]),
    "dnpeff_set_csr_rows": (C.c_int, [_P, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _I32]),
    "dnpeff_set_csr_rows_device": (C.c_int, [_P, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P, _I32]),
    "dnpeff_get_shard": (C.c_int, [_P, C.POINTER(_I32), C.POINTER(_I32), C.POINTER(_I32)]),
    "dnpeff_comm_agree": (C.c_int, [_P, _I32, C.POINTER(_I32)]),
    "dnpeff_run_steps": (C.c_int, [_P, _I32, _I32, _I32]),
    "dnpeff_set_csr_device": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _I32]),
    "dnpeff_set_csr_retain": (C.c_int, [_P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _I64]),
    "dnpeff_get_shape": (C.c_int, [_P] + [C.POINTER(_I64)] * 5),
    "dnpeff_get_layout": (C.c_int, [_P, C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I32), C.POINTER(_I32)]),
    "dnpeff_get_new_to_og": (C.c_int, [_P, _P]),
    "dnpeff_get_shard_columns": (C.c_int, [_P, _P, _P]),
    "dnpeff_export_shard_csr": (C.c_int, [_P, _P, _P, _P]),
    "dnpeff_export_shard_csc": (C.c_int, [_P, _P, _P, _P]),
    "dnpeff_a_sq_norm": (C.c_int, [_P, C.POINTER(C.c_double)]),
    "dnpeff_a_sum": (C.c_int, [_P, C.POINTER(C.c_double)]),
    "dnpeff_init_factors": (C.c_int, [_P, _P, _P]),
    "dnpeff_set_h_csr": (C.c_int, [_P, _P, _P, _P]),
    "dnpeff_set_w_row_offset": (C.c_int, [_P, _I64]),
    "dnpeff_set_init_scale": (C.c_int, [_P, C.c_float]),
    "dnpeff_get_w": (C.c_int, [_P, _P]),
    "dnpeff_get_h": (C.c_int, [_P, _P]),
    "dnpeff_nccl_unique_id": (C.c_int, [_P]),
    "dnpeff_comm_init": (C.c_int, [_P, _P, C.c_int, C.c_int]),
    "dnpeff_step_w": (C.c_int, [_P]),
    "dnpeff_step_h": (C.c_int, [_P]),
    "dnpeff_run": (C.c_int, [_P, _I32, _I32]),
    "dnpeff_synchronize": (C.c_int, [_P]),
    "dnpeff_loss": (C.c_int, [_P, C.POINTER(C.c_double)]),
    "dnpeff_fit_w_only": (C.c_int, [_P, _I32, C.POINTER(C.c_double)]),
    "dnpeff_enable_timing": (C.c_int, [_P, C.c_int]),
    "dnpeff_get_timing": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(_I64)]),
    "dnpeff_launch_count": (C.c_int, [_P, C.POINTER(_I64)]),
    "dnpeff_op_spmm": (C.c_int, [_P, _P, _P, _I64, _P, _I32, _P, _P]),
    "dnpeff_op_gram": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "dnpeff_op_mu_update": (C.c_int, [_P, _P, _P, _I64, _I32, C.c_float, _P]),
    "dnpeff_op_block_product": (C.c_int, [_P, _I64, _I64, _P, _I32, _P, _P]),
    "dnpeff_op_hoyer_project": (C.c_int, [_P, _I64, _I32, C.c_float, C.c_float, _I32, _I32, _P, _P, _P]),
    "dnpeff_sparsify_w": (C.c_int, [_P, C.c_float, C.c_float, _I32, _P, _P]),
    "dnpeff_pef_hdf5_info": (C.c_int, [C.c_char_p] + [C.POINTER(_I64)] * 3),
    "dnpeff_read_pef_hdf5": (C.c_int, [C.c_char_p, _I64, _I64, _P, _P, _P]),
    "dnpeff_load_pef_hdf5": (C.c_int, [_P, C.c_char_p, _I64, _I64, _I32]),
    "dnpeff_save_decomposition_hdf5": (C.c_int, [C.c_char_p, _P, _P, _P, _I64, _I32, _I64, _I64]),
    "dnpeff_decomposition_hdf5_info": (C.c_int, [C.c_char_p, C.POINTER(_I64), C.POINTER(_I32),
                                                 C.POINTER(_I64), C.POINTER(_I64)]),
    "dnpeff_read_decomposition_hdf5": (C.c_int, [C.c_char_p, _P, _P, _P]),
    "dnpeff_save_sparse_decomposition_hdf5": (C.c_int, [C.c_char_p, _P, _I64, _I32, _P, _P, _P, _P, _I64, _I64]),
    "dnpeff_sparse_decomposition_hdf5_info": (C.c_int, [C.c_char_p, _P, _P, _P, _P, _P]),
    "dnpeff_read_sparse_decomposition_hdf5": (C.c_int, [C.c_char_p, _P, _P, _P, _P, _P]),
    "dnpeff_hdf5_dataset_info": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(_I32), C.POINTER(_I64),
                                           C.POINTER(_I32), C.POINTER(_I32)]),
    "dnpeff_hdf5_read_f64": (C.c_int, [C.c_char_p, C.c_char_p, _I64, _I64, _P]),
    "dnpeff_write_pef_hdf5": (C.c_int, [C.c_char_p, _I64, _I64, _P, _P, _P, _I64]),
    "dnpeff_op_gram_noalloc": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "dnpeff_synth_pef_device_rows": (C.c_int, [_I64, _I64, _I64, _I64, C.c_double, C.c_double, C.c_uint64,
                                               _P, _P, _P, _P]),
    "dnpeff_synth_pef_device": (C.c_int, [_I64, _I64, _I64, C.c_double, C.c_double, C.c_uint64,
                                          _P, _P, _P, _P]),
}


def lib():
    """Loads the CUDA library; raises if it has not been built (no fallback)."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise DnpeffError(-2, "libdnpeff.so is not built (run `python -m npeff_ref_b200.build`); "
                                  "there is no CPU fallback")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = handle
    return _LIB


def check(code):
    if code != OK:
        msg = lib().dnpeff_last_error()
        raise DnpeffError(code, msg.decode("utf-8", "replace") if msg else "")
