"""ctypes declarations of the C ABI in include/vmcuda.h, one to one."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvmcuda.so")

VM_OK = 0
VM_ERR_INVALID_ARGUMENT = 1
VM_ERR_UNSUPPORTED_FORMAT = 2
VM_ERR_UNSUPPORTED_LENS = 3
VM_ERR_NETWORK_SHAPE = 4
VM_ERR_CUDA = 5
VM_ERR_OUT_OF_MEMORY = 6
VM_ERR_DEVICE_ABORT = 7
VM_ERR_NO_BSP = 8

VM_RESULTS_ON_DEVICE = 1
VM_TIME_STAGES = 2


class vm_lens(C.Structure):
    _fields_ = [
        ("dimensions", C.c_int32 * 2),
        ("projection", C.c_int32),
        ("focal_length", C.c_float),
        ("centre", C.c_float * 2),
        ("k", C.c_float * 2),
        ("fov", C.c_float),
    ]


class vm_layer(C.Structure):
    _fields_ = [
        ("weights", C.c_void_p),
        ("biases", C.c_void_p),
        ("n_in", C.c_int32),
        ("n_out", C.c_int32),
        ("activation", C.c_int32),
    ]


class vm_frame(C.Structure):
    _fields_ = [
        ("mesh", C.c_void_p),
        ("ranges", C.c_void_p),
        ("n_ranges", C.c_int32),
        ("Hoc", C.c_float * 16),
        ("lens", vm_lens),
        ("image", C.c_void_p),
        ("format", C.c_uint32),
        ("image_on_device", C.c_int32),
    ]


class vm_batch_result(C.Structure):
    _fields_ = [
        ("n_frames", C.c_int32),
        ("n_neighbours", C.c_int32),
        ("n_classes", C.c_int32),
        ("on_device", C.c_int32),
        ("offsets", C.POINTER(C.c_int32)),
        ("pixel_coordinates", C.POINTER(C.c_float)),
        ("global_indices", C.POINTER(C.c_int32)),
        ("neighbourhood", C.POINTER(C.c_int32)),
        ("classifications", C.POINTER(C.c_float)),
    ]


# every symbol the header declares: name -> (restype, argtypes)
SYMBOLS = {
    "vm_engine_create": (C.c_int, [C.c_int, C.POINTER(vm_layer), C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_void_p)]),
    "vm_engine_destroy": (None, [C.c_void_p]),
    "vm_mesh_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_void_p)]),
    "vm_mesh_set_bsp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "vm_mesh_release": (None, [C.c_void_p, C.c_void_p]),
    "vm_run_batch": (C.c_int, [C.c_void_p, C.POINTER(vm_frame), C.c_int32, C.c_uint32, C.POINTER(vm_batch_result)]),
    "vm_project": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(vm_lens),
                             C.POINTER(vm_batch_result)]),
    "vm_classify": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(vm_lens), C.c_void_p,
                              C.c_uint32, C.POINTER(vm_batch_result)]),
    "vm_project_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(vm_lens), C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]),
    "vm_sample": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_uint32, C.c_void_p]),
    "vm_network": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "vm_stage_times": (C.c_int, [C.c_void_p, C.POINTER(C.c_char_p), C.POINTER(C.c_float), C.c_int32,
                                 C.POINTER(C.c_int32)]),
    "vm_timer_start": (C.c_int, [C.c_void_p]),
    "vm_timer_stop": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "vm_set_wait_limit": (C.c_int, [C.c_void_p, C.c_uint32]),
    "vm_launch_count": (C.c_int64, [C.c_void_p]),
    "vm_host_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "vm_host_free": (None, [C.c_void_p]),
    "vm_last_error": (C.c_char_p, []),
    "vm_hostmesh_create": (C.c_int, [C.c_char_p, C.c_char_p, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float,
                                     C.POINTER(C.c_void_p)]),
    "vm_hostmesh_destroy": (None, [C.c_void_p]),
    "vm_hostmesh_n_nodes": (C.c_int32, [C.c_void_p]),
    "vm_hostmesh_n_neighbours": (C.c_int32, [C.c_void_p]),
    "vm_hostmesh_n_bsp": (C.c_int32, [C.c_void_p]),
    "vm_hostmesh_nodes": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "vm_hostmesh_bsp": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "vm_hostmesh_lookup": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(vm_lens), C.c_void_p, C.c_int32,
                                     C.POINTER(C.c_int32)]),
}

_lib = None


def load():
    """Loads libvmcuda.so. There is no fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m visualmesh_b200.build` (there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class VisualMeshError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"vm_status {status}: {message}")
        self.status = status


def check(status):
    if status != VM_OK:
        raise VisualMeshError(status, load().vm_last_error().decode(errors="replace"))
