"""vesta_step_static: the decode step for callers that may not allocate device memory.

Some hosts of this library own every byte of device memory themselves (a plugin inside another
runtime, a serving process that froze its memory plan after start-up), so cudaMalloc, or
any helper that allocates on their behalf, is off the table for them. For those callers the
library keeps the step kernel's work space in a fixed 4 MiB array of its own. This test drives
that entry point through the C ABI next to the ordinary path (whose work space PyTorch allocates)
on the same inputs, two steps in a row, and expects the same logits and tokens.

Collected last on purpose: the entry point shares one array per GPU across all callers, and the
test must hold both in a fresh process and after everything else has run.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import TIGHT

pytestmark = pytest.mark.gpu


def static_step(lib, k, residues, stream, logits_out, next_out, scratch_floats=None, tmaps=None, status_out=None, n_residues=None):
    low = k.lowered
    ptrs = [residues[name].data_ptr() for name, _, _ in low.params]
    arr = (ctypes.c_ulonglong * len(ptrs))(*ptrs)
    lo, _, lshape = low.scratch['logit']
    no, _, nshape = low.scratch['next']
    return lib.vesta_step_static(k.fn, k.grid, k.block, k.smem, len(ptrs) if n_residues is None else n_residues, arr,
                                 ctypes.c_ulonglong(k.WP.data_ptr()), ctypes.c_ulonglong(k.PT.data_ptr()),
                                 ctypes.c_ulonglong(tmaps.data_ptr()),
                                 ctypes.c_size_t(low.scratch_floats if scratch_floats is None else scratch_floats),
                                 ctypes.c_size_t(low.counters),
                                 ctypes.c_size_t(lo), ctypes.c_size_t(int(np.prod(lshape))), ctypes.c_void_p(logits_out.data_ptr()),
                                 ctypes.c_size_t(no), ctypes.c_size_t(int(np.prod(nshape))), ctypes.c_void_p(next_out.data_ptr()),
                                 ctypes.c_void_p(status_out.data_ptr() if status_out is not None else None), ctypes.c_void_p(stream))


def test_static_scratch_step_matches_the_allocating_path():
    from vesta_gpu_b200 import launch
    from vesta_gpu_b200.shapes import TINY3
    from vesta_gpu_b200.synth import SynthGPT2
    from vesta_gpu_b200.gpt2 import VestaGPT2
    lib = launch.lib()
    lib.vesta_step_static.restype = ctypes.c_int
    lib.vesta_static_last_error.restype = ctypes.c_char_p
    lib.vesta_static_scratch_bytes.restype = ctypes.c_size_t
    assert lib.vesta_static_scratch_bytes() == 4 << 20

    B, tmax = 3, 16
    m = VestaGPT2(SynthGPT2(TINY3, 11, 'rich'), batch=B, tmax=tmax)
    m.reset()
    start = torch.tensor([5, 17, 300], dtype=torch.int32, device='cuda')
    m.x.copy_(start)

    # a second set of per-sequence state for the no-allocation path: same weights, own x, t and KV cache
    mine = dict(m.k.keep)
    mine['x'] = start.clone()
    mine['t'] = torch.zeros_like(m.t)
    mine['keys'] = torch.zeros_like(m.keys)
    mine['vals'] = torch.zeros_like(m.vals)
    tmaps = m.k.tensor_maps(mine)                # the caller's own descriptors of its own cache
    logits = torch.empty(B, TINY3.N, dtype=torch.float32, device='cuda')
    nxt = torch.empty(B, dtype=torch.float32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream

    status = torch.full((1,), 77, dtype=torch.int32, device='cuda')
    for step in range(2):                       # two calls in a row: the second one finds the first one's leftovers
        m.step()
        rc = static_step(lib, m.k, mine, stream, logits, nxt, tmaps=tmaps, status_out=status)
        assert rc == 0, lib.vesta_static_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0, step
        assert torch.allclose(logits, m.logits(), atol=TIGHT, rtol=0), step
        assert torch.equal(nxt, m.next()), step
        assert torch.equal(mine['x'], m.x) and torch.equal(mine['t'], m.t), step
        assert torch.equal(mine['keys'], m.keys) or torch.allclose(mine['keys'].float(), m.keys.float(), atol=2e-3)
    m.k.check()

    # a step that needs more work space than the library holds is refused, with a message, and launches nothing
    before = logits.clone()
    rc = static_step(lib, m.k, mine, stream, logits, nxt, scratch_floats=(4 << 20), tmaps=tmaps)
    assert rc != 0 and b'static scratch holds' in lib.vesta_static_last_error()
    torch.cuda.synchronize()
    assert torch.equal(before, logits)
    # sizes that would wrap around a 64-bit byte count are refused as well, and so is an argument list that
    # would not fit the entry point's own array
    rc = static_step(lib, m.k, mine, stream, logits, nxt, scratch_floats=(1 << 62) + 8, tmaps=tmaps)
    assert rc != 0 and b'static scratch holds' in lib.vesta_static_last_error()
    rc = static_step(lib, m.k, mine, stream, logits, nxt, tmaps=tmaps, n_residues=57)
    assert rc != 0 and b'residues' in lib.vesta_static_last_error()

    # a step the kernel itself refuses (the position is the end of the cache) comes back as a status, not as
    # "token 0": the call succeeds, the status word says why nothing was computed, x and t stay as they were
    mine['t'].fill_(tmax)
    x_before = mine['x'].clone()
    rc = static_step(lib, m.k, mine, stream, logits, nxt, tmaps=tmaps, status_out=status)
    assert rc == 0, lib.vesta_static_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) & 0xff00 == 0x900
    assert torch.equal(mine['x'], x_before) and int(mine['t'][0]) == tmax
    # and the next good step through the same array is unaffected by that refusal
    mine['t'].fill_(2)
    rc = static_step(lib, m.k, mine, stream, logits, nxt, tmaps=tmaps, status_out=status)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
