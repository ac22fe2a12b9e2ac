"""Seeded synthetic weights and prompts (stand-ins for the pretrained checkpoint and the
English prompt of the reference benchmark, bench/g0_bench.py:196-200, which need a download).

Weights: N(0, 0.02) for matrices and embeddings, zero biases, unit LayerNorm ('baseline'),
or with non-trivial biases and LayerNorm parameters ('rich', used by parity tests so that a
dropped bias or gain cannot pass). Values are rounded to fp16 once on the CPU; the same bits
go to the GPU and, up-cast to fp32, to the CPU oracle.
"""
import numpy as np

from .shapes import Shape

MATS = ('wte', 'wpe', 'qkvw', 'ow', 'fcw', 'pw')


def weight_shapes(sh: Shape):
    L, D, F, N, J, C = sh.L, sh.D, sh.F, sh.N, sh.J, sh.C
    return dict(wte=(N, D), wpe=(C, D), ln1w=(L, D), ln1b=(L, D), qkvw=(L, D, J), qkvb=(L, J),
                ow=(L, D, D), ob=(L, D), ln2w=(L, D), ln2b=(L, D), fcw=(L, D, F), fcb=(L, F),
                pw=(L, F, D), pb=(L, D), lnfw=(D,), lnfb=(D,))


def make_weights(sh: Shape, seed=0, init='baseline'):
    """-> dict name -> np.float16 array, in the residue layout of the step program"""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, shape in weight_shapes(sh).items():
        if name in MATS:
            w = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        elif name.startswith('ln') and name.endswith('w'):
            w = np.ones(shape, np.float32)
            if init == 'rich':
                w += rng.standard_normal(shape, dtype=np.float32) * np.float32(0.1)
        else:
            w = np.zeros(shape, np.float32)
            if init == 'rich':
                w += rng.standard_normal(shape, dtype=np.float32) * np.float32(0.05)
        out[name] = w.astype(np.float16)
    return out


def make_prompts(sh: Shape, batch, length, seed=1):
    """uniform token ids, (batch, length) int32"""
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, sh.N, size=(batch, length), dtype=np.int64).astype(np.int32)


def make_ragged_prompts(sh: Shape, batch, lo, hi, seed=1):
    """per-sequence prompt lengths uniform in [lo, hi]; -> (lengths int32 [batch], tokens int32 [batch, hi])"""
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = rng.integers(lo, hi + 1, size=batch, dtype=np.int64).astype(np.int32)
    toks = rng.integers(0, sh.N, size=(batch, hi), dtype=np.int64).astype(np.int32)
    return lens, toks


def make_cache(sh: Shape, seed, positions, scale=0.3):
    """a filled KV cache of one sequence: (keys, vals) fp16 [L, positions, H, E], N(0, scale), from a seed.
    Stands for the cache a long prompt would have left, where running the prompt is too slow (the reference
    interpreter needs about a second per position)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    k = (rng.standard_normal((sh.L, positions, sh.H, sh.E), dtype=np.float32) * scale).astype(np.float16)
    v = (rng.standard_normal((sh.L, positions, sh.H, sh.E), dtype=np.float32) * scale).astype(np.float16)
    return k, v


class SynthGPT2:
    """Stands where the Hugging Face model stands in VestaGPT2(hf, ...): offers state_dict()
    under the Hugging Face names (vesta/gpt2.py:18-25), built from make_weights."""

    def __init__(self, sh: Shape, seed=0, init='baseline', weights=None):
        self.shape = sh
        self.weights = weights if weights is not None else make_weights(sh, seed, init)

    def state_dict(self):
        import torch
        w = {k: torch.from_numpy(v) for k, v in self.weights.items()}
        sd = {'transformer.wte.weight': w['wte'], 'transformer.wpe.weight': w['wpe'],
              'transformer.ln_f.weight': w['lnfw'], 'transformer.ln_f.bias': w['lnfb']}
        per = dict(ln1w='ln_1.weight', ln1b='ln_1.bias', qkvw='attn.c_attn.weight', qkvb='attn.c_attn.bias',
                   ow='attn.c_proj.weight', ob='attn.c_proj.bias', ln2w='ln_2.weight', ln2b='ln_2.bias',
                   fcw='mlp.c_fc.weight', fcb='mlp.c_fc.bias', pw='mlp.c_proj.weight', pb='mlp.c_proj.bias')
        for l in range(self.shape.L):
            for k, hn in per.items():
                sd[f'transformer.h.{l}.{hn}'] = w[k][l]
        return sd
