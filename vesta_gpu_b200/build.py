"""Build steps of the package: the C-ABI shared library and ahead-of-time cubins of the step kernel.

    build_library()                      nvcc -> vesta_gpu_b200/libvesta_b200.so (sm_100a)
    prebuild(shape, batch, tmax, ...)    lower + nvcc -cubin for one configuration into the cubin cache
                                         that launch.compile_cubin consults before calling NVRTC

Both run without a GPU (nvcc cross-compiles).
"""
import os
import subprocess
from pathlib import Path

from .shapes import Shape

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
NVCC = os.environ.get('NVCC', '/usr/local/cuda/bin/nvcc')
ARCH_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo']


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError('command failed: ' + ' '.join(map(str, cmd)) + '\n' + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_library(force=False):
    """compile every source under csrc/ that belongs to the shared library"""
    out = HERE / 'libvesta_b200.so'
    srcs = sorted(list((HERE / 'csrc').glob('*.cpp')) + list((HERE / 'csrc').glob('*.cu')))
    newest = max(s.stat().st_mtime for s in srcs + [ROOT / 'include' / 'vesta_b200.h'])
    if out.exists() and out.stat().st_mtime >= newest and not force:
        return out
    cmd = [NVCC, '-O2', '-std=c++17', '-shared', '-Xcompiler', '-fPIC', *ARCH_FLAGS, '-I', str(ROOT / 'include'),
           *map(str, srcs), '-o', str(out), '-ldl']
    run(cmd)
    return out


def residue_spec(sh: Shape, batch, tmax, per_sequence_t=False):
    """residue name -> (shape, dtype) as vesta_gpu_b200.gpt2.VestaGPT2 passes it to lower()"""
    from .synth import weight_shapes
    spec = {'x': ((batch,), 'i32'), 't': (((batch,) if per_sequence_t else ()), 'i32')}
    for k, v in weight_shapes(sh).items():
        spec[k] = (tuple(v), 'f16')
    spec['keys'] = ((batch, sh.L, tmax, sh.H, sh.E), 'f16')
    spec['vals'] = spec['keys']
    return spec


def lower_for(sh: Shape, batch, tmax, feedback=True, timing=False, per_sequence_t=False, grid=148, prompt_len=0, slab_tiles=None, tune=None):
    from .lower import lower
    from .program_text import decode_program
    per_token = ('x', 'keys', 'vals') + (('t',) if per_sequence_t else ())
    return lower(decode_program(sh), residue_spec(sh, batch, tmax, per_sequence_t), {'s': tmax}, batch=batch,
                 per_token=per_token, outputs=('logit', 'next'),
                 feedback={'x': 'next', 't': 1} if feedback else None, timing=timing, grid=grid, prompt_len=prompt_len, slab_tiles=slab_tiles, tune=tune)


def prebuild(sh: Shape, batch, tmax, verbose=False, **kw):
    """nvcc-compile the step kernel of one configuration into the cubin cache; -> (path, ptxas log)"""
    from .launch import ARCH, CUBIN_DIR, _cache_key
    low = lower_for(sh, batch, tmax, **kw)
    CUBIN_DIR.mkdir(exist_ok=True)
    key = _cache_key(low.src, ARCH)
    cu, out = CUBIN_DIR / (key + '.cu'), CUBIN_DIR / (key + '.cubin')
    if out.exists():
        return out, ''
    cu.write_text(low.src)
    log = run([NVCC, '-O3', '-std=c++17', *ARCH_FLAGS, '-Xptxas', '-v', '-cubin', '-o', str(out), str(cu)])
    cu.unlink()
    if verbose:
        print(log)
    return out, log
