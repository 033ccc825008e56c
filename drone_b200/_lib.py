"""ctypes binding of libdrone_b200.so (the C ABI declared in include/drone_b200.h).

Loading fails loudly when the library is missing: there is no CPU or PyTorch
fallback for any entry point.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libdrone_b200.so")

OP_A = 0
OP_AT = 1
PLAN_A = 1
PLAN_AT = 2
PLAN_BOTH = 3


class DroneError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("drone_b200 error %d: %s" % (code, message))
        self.code = code


class PRResponse(C.Structure):
    _fields_ = [("Mirror2MasterSendSize", C.c_int), ("Mirror2MasterRecvSize", C.c_int),
                ("Master2MirrorSendSize", C.c_int), ("Master2MirrorRecvSize", C.c_int),
                ("VisitedSize", C.c_int), ("LocalVertexSize", C.c_int),
                ("CalTime", C.c_float), ("SendTime", C.c_float)]

    def is_empty(self):
        """IsEmpty of the Go bridge, DRONE/src/tools/cuda_convert.go:47-52."""
        return (self.Mirror2MasterSendSize == 0 and self.Mirror2MasterRecvSize == 0 and
                self.Master2MirrorSendSize == 0 and self.Master2MirrorRecvSize == 0)


class SpmmOpts(C.Structure):
    """drone_spmm_opts of include/drone_b200.h."""
    _fields_ = [("epilogue", C.c_int), ("row_class", C.c_int), ("unit_values", C.c_int), ("reserved_", C.c_int),
                ("d_row_scale", C.c_void_p), ("push_up_to", C.c_void_p)]


EPILOGUE_NONE = 0
EPILOGUE_RELU = 1


class PlanStats(C.Structure):
    _fields_ = [
        ("n_rows", C.c_int),
        ("nnz", C.c_int),
        ("short_row_limit", C.c_int),
        ("chunk_nnz", C.c_int),
        ("n_long_rows", C.c_int * 2),
        ("n_chunks", C.c_int * 2),
        ("n_split_rows", C.c_int * 2),
        ("n_partials", C.c_int * 2),
        ("scratch_bytes", C.c_longlong),
        ("last_slice_width", C.c_int),
        ("hot_rows_tagged", C.c_int),
    ]


_lib = None


def _declare(lib):
    vp, i, f, ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
    sigs = {
        "drone_version": (i, []),
        "drone_last_error": (C.c_char_p, []),
        "drone_kernel_launch_count": (ll, []),
        "drone_compute_csr_values": (i, [vp, vp, vp, vp, i, vp, vp]),
        "drone_plan_create": (i, [C.POINTER(vp), i, i, vp, vp, vp, vp, vp, i, vp]),
        "drone_plan_destroy": (i, [vp]),
        "drone_plan_get_stats": (i, [vp, C.POINTER(PlanStats)]),
        "drone_plan_get_csr": (i, [vp, i, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
        "drone_spmm": (i, [vp, i, i, vp, i, vp, i, vp]),
        "drone_plan_reserve": (i, [vp, i, i]),
        "drone_spmm_ex": (i, [vp, i, i, vp, i, vp, i, C.POINTER(SpmmOpts), vp]),
        "drone_degree_scales": (i, [vp, vp, i, vp, vp, vp]),
        "drone_plan_set_row_classes": (i, [vp, vp, i, vp]),
        "drone_spmm_rows": (i, [vp, i, i, i, vp, i, vp, i, vp]),
        "drone_spmm_host": (i, [vp, i, i, vp, vp]),
        "drone_spmm_host_submit": (i, [vp, i, i, vp, vp, C.POINTER(C.c_longlong)]),
        "drone_spmm_host_wait": (i, [vp, C.c_longlong]),
        "drone_spmm_static_scratch": (i, [vp, i, i, vp, i, vp, i, vp]),
        "drone_host_alloc": (i, [C.POINTER(vp), C.c_size_t]),
        "drone_host_free": (i, [vp]),
        "drone_comm_unique_id": (i, [vp, C.c_size_t]),
        "drone_comm_create": (i, [C.POINTER(vp), i, i, vp, C.c_size_t]),
        "drone_comm_adopt": (i, [C.POINTER(vp), vp, i, i]),
        "drone_comm_destroy": (i, [vp]),
        "drone_comm_allreduce_sum": (i, [vp, vp, C.c_size_t, i, vp]),
        "drone_comm_bcast": (i, [vp, vp, C.c_size_t, i, vp]),
        "drone_comm_reduce_sum": (i, [vp, vp, C.c_size_t, i, vp]),
        "drone_clear_mirror_rows": (i, [vp, i, i, i, vp, vp]),
        "drone_xplan_create": (i, [C.POINTER(vp), i, i, i, vp, vp, vp, vp, i]),
        "drone_xplan_destroy": (i, [vp]),
        "drone_xplan_enable_p2p": (i, [vp, vp, vp]),
        "drone_xplan_counts": (i, [vp, vp, vp, C.POINTER(i)]),
        "drone_xplan_lists": (i, [vp, vp, vp]),
        "drone_exchange_sum": (i, [vp, vp, vp, i, i, vp]),
        "drone_exchange_finish": (i, [vp, vp, i, i, vp]),
        "drone_dense_xplan_create": (i, [C.POINTER(vp), i, i, i, vp, i, vp, vp, i]),
        "drone_dense_xplan_destroy": (i, [vp]),
        "drone_dense_xplan_boundary_rows": (ll, [vp]),
        "drone_exchange_sum_dense": (i, [vp, vp, vp, i, i, vp]),
        "drone_exchange_sum_local": (i, [i, C.POINTER(vp), C.POINTER(vp), i, C.POINTER(i), vp]),
        "drone_pr_create": (i, [C.POINTER(vp), i, i, i, vp, vp, vp, vp, vp, vp, i, C.c_double]),
        "drone_pr_destroy": (i, [vp]),
        "drone_pr_peval": (i, [vp, C.POINTER(PRResponse), vp]),
        "drone_pr_inceval": (i, [vp, C.POINTER(PRResponse), vp]),
        "drone_pr_power_iterate": (i, [vp, i, C.c_double, vp]),
        "drone_pr_step_local": (i, [i, C.POINTER(vp), i, C.POINTER(PRResponse), vp]),
        "drone_pr_power_iterate_local": (i, [i, C.POINTER(vp), i, C.c_double, vp]),
        "drone_pr_values": (i, [vp, vp, vp]),
        "drone_pr_set_isolated_count": (i, [vp, ll]),
        "drone_pr_device_arrays": (i, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
        "drone_mp_create": (i, [C.POINTER(vp), i, i, i, vp, vp, vp, vp, vp, vp]),
        "drone_mp_destroy": (i, [vp]),
        "drone_mp_peval": (i, [vp, i, C.POINTER(PRResponse), vp]),
        "drone_mp_inceval": (i, [vp, C.POINTER(PRResponse), vp]),
        "drone_mp_step_local": (i, [i, C.POINTER(vp), i, i, C.POINTER(PRResponse), vp]),
        "drone_mp_values": (i, [vp, vp, vp]),
        "drone_mp_device_arrays": (i, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
        "drone_ebv_partition": (i, [i, ll, vp, vp, i, i, vp, vp, vp, vp, vp]),
        "drone_presence_bits_host": (i, [i, i, vp, vp, vp, vp]),
        "drone_text_ints_count": (i, [C.c_char_p, C.POINTER(ll), C.POINTER(ll)]),
        "drone_text_ints_read": (i, [C.c_char_p, vp, ll, vp, ll, C.POINTER(ll), C.POINTER(ll)]),
        "drone_text_edges_read": (i, [C.c_char_p, vp, vp, ll, C.POINTER(ll)]),
        "drone_partition_write": (i, [C.c_char_p, i, i, vp, vp, vp, vp, vp, vp]),
        "drone_partition_read_header": (i, [C.c_char_p, C.POINTER(i), C.POINTER(i), vp]),
        "drone_partition_read": (i, [C.c_char_p, i, vp, vp, vp, vp, vp]),
        "drone_graph_build_host": (i, [i, i, vp, vp, vp, vp, vp, vp, C.POINTER(i)]),
        "drone_graph_build_device": (i, [i, i, vp, vp, vp, vp, vp, vp, C.POINTER(i), vp]),
        "drone_route_tables_host": (i, [i, vp, vp, vp, vp, i, i, vp, vp, i, vp, vp, vp]),
        "drone_rmat_edges": (i, [i, ll, C.c_ulonglong, C.c_double, C.c_double, C.c_double, ll, vp, vp, vp]),
        "drone_rmat_edges_host": (i, [i, ll, C.c_ulonglong, C.c_double, C.c_double, C.c_double, ll, vp, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib():
    """The loaded library.  Raises if it has not been built (python -m drone_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "drone_b200: %s is missing. Build it with `python -m drone_b200.build`; "
                "there is no fallback path." % LIB_PATH)
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def check(code):
    if code != 0:
        raise DroneError(code, lib().drone_last_error().decode("utf-8", "replace"))
