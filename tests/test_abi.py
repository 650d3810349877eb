"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares, validates its
arguments before touching a device, and refuses to run without a GPU instead of falling back."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from visualmesh_b200 import abi
from visualmesh_b200 import workloads as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "vmcuda.h")).read()
    return sorted(set(re.findall(r"^VM_API [a-z_0-9 \*]+?\b(vm_[a-z_0-9]+)\(", text, flags=re.M)))


def test_library_exports_every_declared_symbol():
    lib = abi.load()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/vmcuda.h but not exported"
    assert sorted(abi.SYMBOLS) == declared, "visualmesh_b200/abi.py and include/vmcuda.h disagree"


def test_struct_layouts_match_the_header():
    assert C.sizeof(abi.vm_lens) == 36
    assert C.sizeof(abi.vm_layer) == 32
    assert C.sizeof(abi.vm_frame) == 136 and abi.vm_frame.image.offset == 120 and abi.vm_frame.lens.offset == 84
    assert C.sizeof(abi.vm_batch_result) == 16 + 5 * 8


def _layers(shapes, acts=None):
    arr = (abi.vm_layer * len(shapes))()
    keep = []
    for i, (n_in, n_out) in enumerate(shapes):
        w, b = np.zeros((n_in, n_out), np.float32), np.zeros((n_out,), np.float32)
        keep += [w, b]
        arr[i].weights, arr[i].biases, arr[i].n_in, arr[i].n_out = w.ctypes.data, b.ctypes.data, n_in, n_out
        arr[i].activation = W.SELU if acts is None else acts[i]
    return arr, keep


@pytest.mark.parametrize("shapes,per_group", [
    ([(27, 8)], [1]),            # 27 is not (N+1) * 4
    ([(28, 8), (9, 2)], [2]),    # dense layer rows != previous width
    ([(28, 8), (40, 2)], [1, 1]),  # second group gathers 5 slots, first 7
    ([(12, 8)], [1]),            # 3 slots: N = 2 is not a mesh
])
def test_network_shape_errors_are_reported_before_any_device_work(shapes, per_group):
    lib = abi.load()
    arr, keep = _layers(shapes)
    lpg = (C.c_int32 * len(per_group))(*per_group)
    out = C.c_void_p()
    status = lib.vm_engine_create(-1, arr, lpg, len(per_group), C.byref(out))
    assert status == abi.VM_ERR_NETWORK_SHAPE
    assert lib.vm_last_error()


def test_unknown_activation_is_rejected():
    lib = abi.load()
    arr, keep = _layers([(28, 8)], acts=[7])
    lpg = (C.c_int32 * 1)(1)
    out = C.c_void_p()
    assert lib.vm_engine_create(-1, arr, lpg, 1, C.byref(out)) == abi.VM_ERR_NETWORK_SHAPE


def test_no_cpu_fallback_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = abi.load()
    arr, keep = _layers([(28, 8)])
    lpg = (C.c_int32 * 1)(1)
    out = C.c_void_p()
    status = lib.vm_engine_create(-1, arr, lpg, 1, C.byref(out))
    assert status == abi.VM_ERR_CUDA and not out.value
    assert b"no CPU fallback" in lib.vm_last_error()
    from visualmesh_b200.engine import Engine, VisualMeshError
    with pytest.raises(VisualMeshError):
        Engine(W.make_network(1, 6, [8, 2]))


def test_null_arguments():
    lib = abi.load()
    assert lib.vm_engine_create(-1, None, None, 1, None) == abi.VM_ERR_INVALID_ARGUMENT
    res = abi.vm_batch_result()
    assert lib.vm_run_batch(None, None, 1, 0, C.byref(res)) == abi.VM_ERR_INVALID_ARGUMENT
    out = C.c_void_p()
    assert lib.vm_hostmesh_create(b"RING7", b"SPHERE", 0.1, 0.0, 1.0, 2.0, 5.0, C.byref(out)) == abi.VM_ERR_INVALID_ARGUMENT
    assert lib.vm_hostmesh_create(b"RING6", b"CUBE", 0.1, 0.0, 1.0, 2.0, 5.0, C.byref(out)) == abi.VM_ERR_INVALID_ARGUMENT
