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


def test_static_step_refuses_oversized_requests_before_touching_the_gpu(built_library):
    """vesta_step_static checks its sizes on the host first: more residues than its argument array holds, a scratch
    size whose byte count would wrap around, and output ranges outside the scratch are all refused with a message
    (no CUDA call has been made at that point, so this runs without a GPU)"""
    lib = ctypes.CDLL(str(built_library))
    lib.vesta_static_last_error.restype = ctypes.c_char_p
    sz, vp, ull = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_ulonglong
    ptrs = (ull * 64)(*([0x1000] * 64))
    fn = vp(0x10)                                   # never launched: every case below is refused before that

    def call(n_res=20, scratch=1024, counters=64, lo=0, ln=16, no=16, nn=4):
        return lib.vesta_step_static(fn, 148, 288, 0, n_res, ptrs, ull(0), ull(0), ull(0), sz(scratch), sz(counters),
                                     sz(lo), sz(ln), vp(None), sz(no), sz(nn), vp(None), vp(None), vp(None))
    assert call(n_res=57) != 0 and b'residues' in lib.vesta_static_last_error()
    assert call(n_res=-1) != 0
    assert call(scratch=(1 << 62) + 8) != 0 and b'static scratch holds' in lib.vesta_static_last_error()
    assert call(scratch=(4 << 20) // 4) != 0 and b'static scratch holds' in lib.vesta_static_last_error()
    assert call(counters=1 << 20) != 0 and b'counter' in lib.vesta_static_last_error()
    assert call(lo=(1 << 64) - 8, ln=16) != 0 and b'output range' in lib.vesta_static_last_error()
    assert call(no=1000, nn=100) != 0 and b'output range' in lib.vesta_static_last_error()
