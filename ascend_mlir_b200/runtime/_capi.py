"""ctypes binding of libAFIRRuntimeCAPI.so (prototypes of include/CAPI/Runtime.h and RuntimeCuda.h)."""
import ctypes

from .utils import find_afirt_capi_lib

_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_vpp = ctypes.POINTER(ctypes.c_void_p)
_szp = ctypes.POINTER(ctypes.c_size_t)

_RUN_TAIL = [ctypes.c_char_p, ctypes.c_int, _vpp, _szp, ctypes.c_int, _vpp, _szp, _u8p, ctypes.c_size_t,
             ctypes.c_int, ctypes.c_uint32]

EXPORTS = [
    "afirt_compiler_create", "afirt_compiler_destroy", "afirt_compiler_compile",
    "afirt_executor_create", "afirt_executor_destroy", "afirt_executor_initialize",
    "afirt_executor_run", "afirt_executor_run_file",
    "afirt_executor_launch_device", "afirt_executor_synchronize", "afirt_executor_workspace_bytes",
    "afirt_executor_last_launch_count", "afirt_executor_total_launch_count", "afirt_executor_last_launch_generated",
    "afirt_runtime_version",
    "afirt_bcast_add_rowsum_no_alloc",
    "afirt_rowsum_exchange_create", "afirt_rowsum_exchange_connect", "afirt_bcast_add_rowsum_exchange",
    "afirt_bcast_add_rowsum_exchange_batch",
    "afirt_rowsum_exchange_status", "afirt_rowsum_exchange_destroy", "afirt_executor_launch_device_exchange",
    "afirt_executor_launch_device_sharded_table", "afirt_peer_export", "afirt_peer_import", "afirt_peer_release",
]

PEER_HANDLE_BYTES = 96  # AFIRT_PEER_HANDLE_BYTES

EXCHANGE_HANDLE_BYTES = 96  # AFIRT_EXCHANGE_HANDLE_BYTES


def get_lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    lib = ctypes.CDLL(str(find_afirt_capi_lib()))
    lib.afirt_compiler_create.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    lib.afirt_compiler_create.restype = ctypes.c_void_p
    lib.afirt_compiler_destroy.argtypes = [ctypes.c_void_p]
    lib.afirt_compiler_destroy.restype = None
    lib.afirt_compiler_compile.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p,
                                           ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_compiler_compile.restype = ctypes.c_int
    lib.afirt_executor_create.argtypes = []
    lib.afirt_executor_create.restype = ctypes.c_void_p
    lib.afirt_executor_destroy.argtypes = [ctypes.c_void_p]
    lib.afirt_executor_destroy.restype = None
    lib.afirt_executor_initialize.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_executor_initialize.restype = ctypes.c_int
    lib.afirt_executor_run.argtypes = [ctypes.c_void_p, _u8p, ctypes.c_size_t] + _RUN_TAIL + [ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_executor_run.restype = ctypes.c_int
    lib.afirt_executor_run_file.argtypes = [ctypes.c_void_p, ctypes.c_char_p] + _RUN_TAIL + [ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_executor_run_file.restype = ctypes.c_int
    lib.afirt_executor_launch_device.argtypes = ([ctypes.c_void_p, _u8p, ctypes.c_size_t] + _RUN_TAIL +
                                                 [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                                  ctypes.c_char_p, ctypes.c_size_t])
    lib.afirt_executor_launch_device.restype = ctypes.c_int
    lib.afirt_executor_launch_device_exchange.argtypes = ([ctypes.c_void_p, _u8p, ctypes.c_size_t] + _RUN_TAIL +
                                                          [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p,
                                                           ctypes.c_char_p, ctypes.c_size_t])
    lib.afirt_executor_launch_device_exchange.restype = ctypes.c_int
    lib.afirt_executor_synchronize.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_executor_synchronize.restype = ctypes.c_int
    lib.afirt_executor_workspace_bytes.argtypes = [ctypes.c_void_p, _u8p, ctypes.c_size_t, _u8p, ctypes.c_size_t,
                                                   _szp, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_executor_workspace_bytes.restype = ctypes.c_int
    lib.afirt_executor_last_launch_count.argtypes = [ctypes.c_void_p]
    lib.afirt_executor_last_launch_count.restype = ctypes.c_int
    lib.afirt_executor_last_launch_generated.argtypes = [ctypes.c_void_p]
    lib.afirt_executor_last_launch_generated.restype = ctypes.c_int
    lib.afirt_executor_total_launch_count.argtypes = [ctypes.c_void_p]
    lib.afirt_executor_total_launch_count.restype = ctypes.c_uint64
    lib.afirt_bcast_add_rowsum_no_alloc.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                                    ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int,
                                                    ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_bcast_add_rowsum_no_alloc.restype = ctypes.c_int
    lib.afirt_executor_launch_device_sharded_table.argtypes = ([ctypes.c_void_p, _u8p, ctypes.c_size_t] + _RUN_TAIL +
                                                               [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int, _vpp,
                                                                ctypes.c_int64, ctypes.c_char_p, ctypes.c_size_t])
    lib.afirt_executor_launch_device_sharded_table.restype = ctypes.c_int
    lib.afirt_peer_export.argtypes = [ctypes.c_void_p, _u8p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_peer_export.restype = ctypes.c_int
    lib.afirt_peer_import.argtypes = [ctypes.c_int, _u8p, _vpp, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_peer_import.restype = ctypes.c_int
    lib.afirt_peer_release.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_peer_release.restype = ctypes.c_int
    lib.afirt_rowsum_exchange_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int64, _vpp, _u8p,
                                                 ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_rowsum_exchange_create.restype = ctypes.c_int
    lib.afirt_rowsum_exchange_connect.argtypes = [ctypes.c_void_p, _u8p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_rowsum_exchange_connect.restype = ctypes.c_int
    lib.afirt_bcast_add_rowsum_exchange.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                                    ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                    ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_bcast_add_rowsum_exchange.restype = ctypes.c_int
    lib.afirt_bcast_add_rowsum_exchange_batch.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, _vpp, _vpp, _vpp,
                                                          ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p,
                                                          ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_bcast_add_rowsum_exchange_batch.restype = ctypes.c_int
    lib.afirt_rowsum_exchange_status.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    lib.afirt_rowsum_exchange_status.restype = ctypes.c_int
    lib.afirt_rowsum_exchange_destroy.argtypes = [ctypes.c_void_p]
    lib.afirt_rowsum_exchange_destroy.restype = None
    lib.afirt_runtime_version.argtypes = []
    lib.afirt_runtime_version.restype = ctypes.c_char_p
    _lib = lib
    return lib
