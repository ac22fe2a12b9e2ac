"""Compile a Lowered program with NVRTC for sm_100a and run it as one cooperative launch per
decode step, through the C ABI of libvesta_b200.so (include/vesta_b200.h) bound with ctypes.

Mirrors the reference run-time (vesta/launch.py:10-73): `TORCH_DT`, `ok`, `compile_cubin`,
and `Kernel` with `view`, `bind`, `launch`, `__call__` and the attributes `mod, fn, smem, sms,
grid, block, lowered, S, bar, TS, args, keep`. PyTorch only allocates buffers and provides the
context and the current stream. There is no fallback: without the shared library, a GPU driver
or NVRTC every call raises.
"""
import ctypes
import hashlib
import os
from pathlib import Path

import numpy as np
import torch

TORCH_DT = {'f32': torch.float32, 'f16': torch.float16, 'i32': torch.int32}
ARCH = 'sm_100a'
HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / 'libvesta_b200.so'
CUBIN_DIR = HERE / '_cubin'

_lib = None


def lib():
    """the C ABI, loaded once"""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f'{LIB_PATH} is missing: build it with `python -c "import __graft_entry__ as g; g.build()"` '
                               '(vesta_gpu_b200.build.build_library)')
        L = ctypes.CDLL(str(LIB_PATH))
        vp, ci, cu, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_size_t
        L.vesta_last_error.restype = ctypes.c_char_p
        L.vesta_rt_version.restype = ci
        L.vesta_set_nvrtc_path.argtypes = [ctypes.c_char_p]
        L.vesta_nvrtc_compile.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ctypes.c_char_p), ci,
                                          ctypes.POINTER(vp), ctypes.POINTER(sz), ctypes.POINTER(vp)]
        L.vesta_free.argtypes = [vp]
        L.vesta_free.restype = None
        L.vesta_init.argtypes = [ci]
        L.vesta_module_load.argtypes = [vp, ctypes.POINTER(vp)]
        L.vesta_module_unload.argtypes = [vp]
        L.vesta_module_get_function.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(vp)]
        L.vesta_func_set_max_dynamic_smem.argtypes = [vp, ci]
        L.vesta_occupancy.argtypes = [vp, ci, sz, ctypes.POINTER(ci)]
        L.vesta_launch_cooperative.argtypes = [vp, cu, cu, cu, vp, ctypes.POINTER(vp)]
        L.vesta_launch.argtypes = [vp, cu, cu, cu, vp, ctypes.POINTER(vp)]
        L.vesta_step_bind.argtypes = [vp, cu, cu, cu, ci, ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(vp)]
        L.vesta_step_run.argtypes = [vp, vp, ci]
        L.vesta_step_run_fused.argtypes = [vp, vp, ci, ci]
        L.vesta_tensor_map_rows.argtypes = [vp, vp, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_uint, ctypes.c_uint]
        L.vesta_step_host.argtypes = [vp, vp, ctypes.c_ulonglong, vp, sz, ctypes.c_ulonglong, vp, sz]
        L.vesta_step_release.argtypes = [vp]
        L.vesta_step_release.restype = None
        _lib = L
    return _lib


def ok(r):
    """raise RuntimeError on a non-zero status of the C ABI (vesta/launch.py:12-15)"""
    if int(r) != 0:
        raise RuntimeError(f'{int(r)}: {lib().vesta_last_error().decode(errors="replace")}')
    return r


def _cache_key(src, arch):
    return hashlib.sha256((arch + '\n' + src).encode()).hexdigest()[:24]


def compile_cubin(src, arch=ARCH, cache=True):
    """source text -> cubin bytes, by NVRTC. Cubins are cached in-tree by a hash of the source
    (the cache is filled ahead of time for the benchmark shapes by vesta_gpu_b200.build)."""
    path = CUBIN_DIR / (_cache_key(src, arch) + '.cubin')
    if cache and path.exists():
        return path.read_bytes()
    L = lib()
    cubin, size, log = ctypes.c_void_p(), ctypes.c_size_t(), ctypes.c_void_p()
    r = L.vesta_nvrtc_compile(src.encode(), arch.encode(), None, 0, ctypes.byref(cubin), ctypes.byref(size),
                              ctypes.byref(log))
    text = ctypes.string_at(log.value).decode(errors='replace') if log.value else ''
    if log.value:
        L.vesta_free(log)
    if r != 0:
        raise RuntimeError('NVRTC failed:\n' + (text or L.vesta_last_error().decode(errors='replace')))
    data = ctypes.string_at(cubin.value, size.value)
    L.vesta_free(cubin)
    if cache:
        try:
            CUBIN_DIR.mkdir(exist_ok=True)
            tmp = path.with_suffix(f'.tmp{os.getpid()}')
            tmp.write_bytes(data)
            os.replace(tmp, path)
        except OSError:
            pass
    return data


STATUS_WHERE = {0x100: 'grid barrier', 0x200: 'weight stream (producer)', 0x300: 'weight stream (consumer)', 0x400: 'step flag', 0x500: 'K/V tile', 0x600: 'logits operand', 0x700: 'tensor-core tile', 0x800: 'K/V stage (producer)',
                0x900: 'token or position out of range', 0xA00: 'exchange between CTAs (tagged values)'}


class Kernel:
    """One lowered program on one GPU: compiled, resident one CTA per SM, launched cooperatively."""

    def __init__(self, lowered, block=None, device=None, blocks_per_sm=None):
        if not torch.cuda.is_available():
            raise RuntimeError('vesta_gpu_b200 needs a CUDA device; there is no CPU path')
        if device is None:
            device = torch.cuda.current_device()
        self.device = torch.device('cuda', device)
        torch.cuda.init()
        with torch.cuda.device(self.device):
            torch.zeros(1, device=self.device)                   # make torch's context current
            L = lib()
            ok(L.vesta_init(device))
            major, minor = torch.cuda.get_device_capability(device)
            if (major, minor) != (10, 0):
                raise RuntimeError(f'this backend is written for sm_100a (B200); device is sm_{major}{minor}')
            self.sms = torch.cuda.get_device_properties(device).multi_processor_count
            if lowered.grid != self.sms:
                raise RuntimeError(f'program was placed for {lowered.grid} SMs, device has {self.sms}: '
                                   f'call lower(..., grid={self.sms})')
            self.lowered = lowered
            self.cubin = compile_cubin(lowered.src, ARCH)
            self._cubin_buf = ctypes.create_string_buffer(self.cubin, len(self.cubin))
            mod, fn, pk = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
            ok(L.vesta_module_load(ctypes.cast(self._cubin_buf, ctypes.c_void_p), ctypes.byref(mod)))
            ok(L.vesta_module_get_function(mod, b'vesta_step', ctypes.byref(fn)))
            ok(L.vesta_module_get_function(mod, b'vesta_pack', ctypes.byref(pk)))
            self.mod, self.fn, self.pack_fn = mod, fn, pk
            self.smem = lowered.shared_bytes
            # The reference's signature defaults to block=256 (vesta/launch.py:30) and callers pass it along: 256 and
            # None both mean "the block size the program was lowered for" (8 consumer warps + the producer warp).
            if block not in (None, 256, lowered.block):
                raise RuntimeError(f'the step kernel runs with {lowered.block} threads per block, not {block}')
            self.block = lowered.block
            if blocks_per_sm not in (None, 1):
                import warnings
                warnings.warn(f'blocks_per_sm={blocks_per_sm} is ignored: the step kernel is placed for one persistent block per SM',
                              RuntimeWarning, stacklevel=2)
            ok(L.vesta_func_set_max_dynamic_smem(fn, self.smem))
            per_sm = ctypes.c_int()
            ok(L.vesta_occupancy(fn, self.block, self.smem, ctypes.byref(per_sm)))
            if per_sm.value < 1:
                raise RuntimeError('kernel cannot be resident at this block size')
            self.grid = self.sms                                 # one persistent CTA per SM
            self.S = torch.zeros(lowered.scratch_floats, dtype=torch.float32, device=self.device)
            self.bar = torch.zeros(lowered.counters, dtype=torch.int32, device=self.device)
            self.TS = torch.zeros(2048, dtype=torch.int64, device=self.device)
            self.PT = torch.from_numpy(np.ascontiguousarray(lowered.place)).to(self.device)
            self.WP = torch.empty(max(lowered.packed_bytes, 512), dtype=torch.uint8, device=self.device)
            self.args, self.keep, self._bound = None, None, None
            self.fuse = 16                                       # decode steps per launch in launch(steps > 1)
            self.feeds_back = '#define V_FEEDBACK 1' in lowered.src
            self.launches = 0

    def view(self, name):
        off, _, shape = self.lowered.scratch[name]
        n = 1
        for s in shape:
            n *= s
        return self.S[off:off + max(1, n)].view(*shape) if shape else self.S[off]

    _host_key = None

    def bind(self, residue):
        """fix the argument list once (launches then cost one call) and pack the weights"""
        L = lib()
        vals = []
        if any(name == '_zeros' for name, _, _ in self.lowered.params) and '_zeros' not in residue:
            # additive parameters the program does not have (lower.OPTIONAL_TERMS): the kernel reads zeros for them
            residue = dict(residue, _zeros=torch.zeros(self.lowered.dims['zeros_len'], dtype=torch.float16, device=self.device))
        for name, dt, _ in self.lowered.params:
            t = residue[name]
            assert t.is_cuda and t.dtype == TORCH_DT[dt] and t.is_contiguous(), (name, t.dtype, dt)
            assert t.device == self.device, (name, t.device)
            vals.append(t.data_ptr())
        self.TM = self.tensor_maps(residue)
        vals += [self.S.data_ptr(), self.bar.data_ptr(), self.TS.data_ptr(), self.WP.data_ptr(), self.PT.data_ptr(), self.TM.data_ptr(), 1]
        self.args = (tuple(vals), tuple([ctypes.c_void_p] * len(vals)))
        self.keep = residue
        if self._bound:
            L.vesta_step_release(self._bound)
        arr = (ctypes.c_ulonglong * len(vals))(*vals)
        bound = ctypes.c_void_p()
        ok(L.vesta_step_bind(self.fn, self.grid, self.block, self.smem, len(vals), arr, ctypes.byref(bound)))
        self._bound = bound
        self.pack(residue)

    def tensor_maps(self, residue):
        """the TMA descriptors of the step kernel, in device memory: the caches as the attention phase reads
        them (K and V with boxes of 32, 64, 96 and 128 rows of one head), then the embedding table in boxes of
        128 rows x 64 columns for the tensor-core logits (vesta_tensor_map_rows)"""
        d = self.lowered.dims
        host = torch.zeros(9 * 128, dtype=torch.uint8)
        for q, rows in enumerate((32, 64, 96, 128)):
            for j, role in enumerate(('keys', 'vals')):
                t = residue[self.lowered.roles[role]]
                ok(lib().vesta_tensor_map_rows(ctypes.c_void_p(host.data_ptr() + 128 * (2 * q + j)), ctypes.c_void_p(t.data_ptr()),
                                               d['D'], d['tmax'], t.shape[0] * d['L'], 64, rows))
        wte = residue[self.lowered.roles['wte']]
        ok(lib().vesta_tensor_map_rows(ctypes.c_void_p(host.data_ptr() + 128 * 8), ctypes.c_void_p(wte.data_ptr()),
                                       d['D'], d['N'], 1, 64, 128))
        return host.to(self.device)

    def pack(self, residue=None):
        """(re)build the packed weight streams from the bound weights; call again after changing them"""
        residue = residue or self.keep
        L = lib()
        vals = [residue[n].data_ptr() for n in self.lowered.pack_params] + [self.WP.data_ptr(), self.PT.data_ptr()]
        store = (ctypes.c_ulonglong * len(vals))(*vals)
        ptrs = (ctypes.c_void_p * len(vals))(*[ctypes.addressof(store) + 8 * i for i in range(len(vals))])
        nblk = self.grid * (self.lowered.dims['L'] + 1)
        with torch.cuda.device(self.device):
            ok(L.vesta_launch(self.pack_fn, nblk, 256, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), ptrs))

    def launch(self, steps=1, per_launch=None):
        """`steps` decode steps on the current stream. With feedback on, up to `per_launch` steps (default
        Kernel.fuse) run inside one launch: the kernel feeds its own token and position between them, which saves
        the gap between launches; without feedback every step is its own launch."""
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        per = per_launch or self.fuse
        if steps > 1 and per > 1 and self.feeds_back:
            ok(lib().vesta_step_run_fused(self._bound, stream, steps, per))
            self.launches += -(-steps // per)
        else:
            ok(lib().vesta_step_run(self._bound, stream, steps))
            self.launches += steps

    def step_host(self, x_dev, tokens_host, result_dev, result_host):
        """one decode step with host buffers: tokens_host (pinned) -> x_dev, one launch, result_dev -> result_host
        (pinned), stream synchronised on return: a single call into the library (vesta_step_host)"""
        # (a host loop calls this once per step: the argument list is kept for the buffers of the last call, the stream
        # handle comes from torch's raw accessor)
        key = (x_dev.data_ptr(), tokens_host.data_ptr(), result_dev.data_ptr(), result_host.data_ptr(), tokens_host.numel(), result_host.numel())
        if self._host_key != key:
            self._host_key = key
            self._host_args = (ctypes.c_ulonglong(key[0]), ctypes.c_void_p(key[1]), ctypes.c_size_t(tokens_host.numel() * tokens_host.element_size()),
                               ctypes.c_ulonglong(key[2]), ctypes.c_void_p(key[3]), ctypes.c_size_t(result_host.numel() * result_host.element_size()))
            self._host_fn = lib().vesta_step_host
        raw = getattr(torch._C, '_cuda_getCurrentRawStream', None)
        stream = raw(self.device.index) if raw else torch.cuda.current_stream(self.device).cuda_stream
        r = self._host_fn(self._bound, ctypes.c_void_p(stream), *self._host_args)
        if r:
            ok(r)
        self.launches += 1

    def __call__(self, residue):
        self.bind(residue)
        self.launch()

    def status(self):
        """0 if every launch so far ran to its end; otherwise a description of the first failure
        (synchronises)"""
        v = int(self.bar[0].item())
        if v == 0:
            return 0
        return f'{STATUS_WHERE.get(v & 0xff00, hex(v & 0xffff))} (CTA {v >> 16})'

    def check(self):
        s = self.status()
        if s:
            raise RuntimeError(f'vesta_step gave up: {s}')

    def clear_status(self):
        """forget a refused step or an abandoned wait: status word, abort flag and the barrier counters back to zero.
        Both are sticky: until this is called every further launch returns at once without touching x, t or the cache
        (a refused step never wrote anything; a launch in which a wait ran out may have written part of a step, so
        reset or reload the decode state before going on)."""
        self.bar.zero_()

    def __del__(self):
        try:
            if getattr(self, '_bound', None):
                lib().vesta_step_release(self._bound)
        except Exception:
            pass
