"""The C ABI (include/vesta_b200.h, libvesta_b200.so): loads without a GPU, exports every declared
symbol, reports errors through its status + message convention. No GPU compute here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'vesta_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(vesta_\w+)\s*\(', text)))


def test_header_declares_the_launch_path():
    names = declared_symbols()
    for need in ('vesta_nvrtc_compile', 'vesta_module_load', 'vesta_module_get_function',
                 'vesta_func_set_max_dynamic_smem', 'vesta_occupancy', 'vesta_launch_cooperative',
                 'vesta_step_bind', 'vesta_step_run', 'vesta_last_error'):
        assert need in names


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(str(built_library))
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.vesta_rt_version() == 1


def test_error_convention(built_library):
    from vesta_gpu_b200 import launch
    L = launch.lib()
    mod = ctypes.c_void_p()
    assert L.vesta_module_load(None, ctypes.byref(mod)) != 0
    assert b'null' in L.vesta_last_error()
    with pytest.raises(RuntimeError):
        launch.ok(L.vesta_step_run(None, None, 1))
    bound = ctypes.c_void_p()
    assert L.vesta_step_bind(None, 1, 1, 0, 0, None, ctypes.byref(bound)) != 0


def test_nvrtc_through_the_abi_without_a_gpu(built_library):
    from vesta_gpu_b200 import launch
    cubin = launch.compile_cubin('extern "C" __global__ void k(float* p) { p[threadIdx.x] = 1.f; }', cache=False)
    assert cubin[:4] == b'\x7fELF'
    with pytest.raises(RuntimeError) as err:
        launch.compile_cubin('extern "C" __global__ void k(float* p) { p[0] = undefined_name; }', cache=False)
    assert 'undefined_name' in str(err.value)          # the compiler log is in the message (vesta/launch.py:21-24)


def test_step_kernel_compiles_for_sm_100a(built_library):
    from vesta_gpu_b200 import launch
    from vesta_gpu_b200.build import lower_for
    from vesta_gpu_b200.shapes import TINY
    for kw in (dict(), dict(per_sequence_t=True), dict(timing=1), dict(feedback=False)):
        low = lower_for(TINY, 3, 17, **kw)
        assert launch.compile_cubin(low.src, cache=False)[:4] == b'\x7fELF'


def test_no_cpu_path():
    """without a CUDA device the product refuses to run instead of falling back"""
    import torch
    if torch.cuda.is_available():
        pytest.skip('a GPU is present')
    from vesta_gpu_b200.launch import Kernel
    from vesta_gpu_b200.build import lower_for
    from vesta_gpu_b200.shapes import TINY
    with pytest.raises(RuntimeError):
        Kernel(lower_for(TINY, 1, 8))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, 'vesta_gpu_b200')
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(('.py', '.cuh', '.cpp', '.cu')):
                text = open(os.path.join(dirpath, f), encoding='utf-8').read()
                assert 'import oracle' not in text and 'from oracle' not in text, f
