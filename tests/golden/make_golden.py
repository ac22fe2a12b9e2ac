"""Generate the golden fixtures in this directory from the reference interpreter itself.

Runs where a checkout of the reference is available (its directory in the environment variable
VESTA_REFERENCE): imports
vesta.interp.run unmodified and drives it exactly as a user would, one sequence at a time,
with fp16-rounded weights up-cast to float32 and np.float16 K/V arrays. The fixtures pin the
CPU oracle (oracle/gpt2_numpy.py) and, through it and directly, the GPU kernel.

    python tests/golden/make_golden.py tiny tiny3 small_rich      # seconds to a minute
    python tests/golden/make_golden.py cfg2                       # 8 processes x 384 steps (sequence 0 is the batch-1 config)
    python tests/golden/make_golden.py xl                         # 8 steps of the XL-shaped program
    python tests/golden/make_golden.py cfg3_sample                # 4 of 64 sequences, 2 steps at context 600 on a seeded cache
    python tests/golden/make_golden.py cfg5_sample                # 4 of 32 sequences with contexts 64..512 (ragged batch)
    python tests/golden/make_golden.py xl16_sample                # 2 of 16 sequences of the XL shape at context 300
    python tests/golden/make_golden.py cfg5_b64_sample cfg5_b256_sample   # 4 sequences of ragged batches of 64 and of 256
    python tests/golden/make_golden.py cfg3_tail_sample           # batch 64 at context 1021..1023: the last position of a 1024-row cache
    python tests/golden/make_golden.py xl1_sample                 # the XL shape at batch 1, context 300

Each fixture: per sequence the greedy token chosen at every step, the top-1 margin, and for a
set of kept steps a strided sample of the logits plus the top-5 (index, value) pairs; small
shapes keep full logits.
"""
import os
import sys
import time
from multiprocessing import Pool

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get('VESTA_REFERENCE')
if not REF:
    raise SystemExit('set VESTA_REFERENCE to a checkout of the reference (the directory that holds vesta/interp.py)')
sys.path.insert(0, ROOT)

from vesta_gpu_b200.shapes import SHAPES                      # noqa: E402
from vesta_gpu_b200.synth import make_weights, make_prompts, make_cache   # noqa: E402
from vesta_gpu_b200.program_text import decode_program        # noqa: E402

STRIDE = 127


def ref_run():
    sys.path.insert(0, REF)
    from vesta.interp import run
    return run


def ref_decode(job):
    """free-running greedy decode of one sequence through vesta.interp.run"""
    shape, seed, init, prompt, gen, keep, full = job
    run = ref_run()
    sh = SHAPES[shape]
    text = decode_program(sh)
    W = {k: v.astype(np.float32) for k, v in make_weights(sh, seed, init).items()}
    steps = len(prompt) + gen
    keys = np.zeros((sh.L, steps, sh.H, sh.E), np.float16)
    vals = np.zeros_like(keys)
    toks, margins, kept = [], [], {}
    x = int(prompt[0])
    for t in range(steps):
        res = dict(W, x=x, t=t, keys=keys, vals=vals)
        env = run(text, res)
        logit = np.asarray(env['logit'][0], np.float32)
        nxt = int(env['next'][0])
        p = np.partition(logit, -2)
        toks.append(nxt); margins.append(float(p[-1] - p[-2]))
        if t in keep:
            top = np.argsort(-logit, kind='stable')[:5]
            kept[t] = (logit.copy() if full else logit[::STRIDE].copy(), top.astype(np.int32), logit[top])
        x = int(prompt[t + 1]) if t + 1 < len(prompt) else nxt
    return np.array(toks, np.int32), np.array(margins, np.float32), kept


def save(name, shape, seed, init, prompts, gen, keep, results, full):
    out = dict(shape=shape, seed=seed, init=init, prompts=prompts, gen=gen, keep=np.array(sorted(keep), np.int32),
               stride=np.int32(1 if full else STRIDE))
    for i, (toks, margins, kept) in enumerate(results):
        out[f'tokens_{i}'] = toks
        out[f'margins_{i}'] = margins
        out[f'logits_{i}'] = np.stack([kept[t][0] for t in sorted(keep)])
        out[f'top_idx_{i}'] = np.stack([kept[t][1] for t in sorted(keep)])
        out[f'top_val_{i}'] = np.stack([kept[t][2] for t in sorted(keep)])
    path = os.path.join(HERE, name + '.npz')
    np.savez_compressed(path, **out)
    print(name, 'written', os.path.getsize(path), 'bytes')


def build(name, shape, seed, init, batch, P, gen, keep, full, procs, pseed=1):
    sh = SHAPES[shape]
    prompts = make_prompts(sh, batch, P, seed=pseed)
    jobs = [(shape, seed, init, prompts[i], gen, keep, full) for i in range(batch)]
    t0 = time.time()
    if procs > 1:
        with Pool(procs) as pool:
            results = pool.map(ref_decode, jobs)
    else:
        results = [ref_decode(j) for j in jobs]
    print(name, 'took %.1f s' % (time.time() - t0))
    save(name, shape, seed, init, prompts, gen, keep, results, full)


def spread(steps, P):
    """kept steps: the first, around the prompt end, a few in the middle, the last"""
    s = {0, 1, P - 2, P - 1, P, P + 1, steps - 2, steps - 1}
    s |= {int(v) for v in np.linspace(2, steps - 3, 8)}
    return {v for v in s if 0 <= v < steps}


def ref_steps_on_cache(job):
    """teacher-forced steps of one sequence on a seeded, filled cache (synth.make_cache): what the batch-64 config
    looks like deep into its context, without the hours the interpreter would need to get there"""
    shape, seed, init, cache_seed, ctx, x0, steps = job
    run = ref_run()
    sh = SHAPES[shape]
    text = decode_program(sh)
    W = {k: v.astype(np.float32) for k, v in make_weights(sh, seed, init).items()}
    k0, v0 = make_cache(sh, cache_seed, ctx)
    keys = np.zeros((sh.L, ctx + steps, sh.H, sh.E), np.float16); vals = np.zeros_like(keys)
    keys[:, :ctx] = k0; vals[:, :ctx] = v0
    x, out = int(x0), []
    for i in range(steps):
        env = run(text, dict(W, x=x, t=ctx + i, keys=keys, vals=vals))
        logit = np.asarray(env['logit'][0], np.float32)
        nxt = int(env['next'][0])
        p = np.partition(logit, -2)
        top = np.argsort(-logit, kind='stable')[:5]
        out.append((x, nxt, float(p[-1] - p[-2]), logit[::STRIDE].copy(), top.astype(np.int32), logit[top]))
        x = nxt
    return out


def build_cache_sample(name, shape, seed, init, batch, ctx, steps, sample):
    """ctx: one context for every sequence, or a function of the sequence index (ragged batch)"""
    sh = SHAPES[shape]
    ctxs = [int(ctx(b)) if callable(ctx) else int(ctx) for b in range(batch)]
    x0 = [(b * 97 + 11) % sh.N for b in range(batch)]
    t0 = time.time()
    with Pool(len(sample)) as pool:
        res = pool.map(ref_steps_on_cache, [(shape, seed, init, 1000 + b, ctxs[b], x0[b], steps) for b in sample])
    print(name, 'took %.1f s' % (time.time() - t0))
    out = dict(shape=shape, seed=seed, init=init, batch=batch, ctx=max(ctxs), ctxs=np.array(ctxs, np.int32), steps=steps, sample=np.array(sample, np.int32),
               x0=np.array(x0, np.int32), cache_seed_base=np.int32(1000), stride=np.int32(STRIDE))
    for i, r in enumerate(res):
        out[f'fed_{i}'] = np.array([s[0] for s in r], np.int32)
        out[f'tokens_{i}'] = np.array([s[1] for s in r], np.int32)
        out[f'margins_{i}'] = np.array([s[2] for s in r], np.float32)
        out[f'logits_{i}'] = np.stack([s[3] for s in r])
        out[f'top_idx_{i}'] = np.stack([s[4] for s in r])
        out[f'top_val_{i}'] = np.stack([s[5] for s in r])
    path = os.path.join(HERE, name + '.npz')
    np.savez_compressed(path, **out)
    print(name, 'written', os.path.getsize(path), 'bytes')


TARGETS = {
    'cfg3_sample': lambda: build_cache_sample('gpt2_cfg3_sample', 'gpt2', 5, 'rich', 64, 600, 2, [0, 21, 42, 63]),
    'xl16_sample': lambda: build_cache_sample('gpt2_xl16_sample', 'gpt2_xl', 0, 'baseline', 16, 300, 2, [0, 15]),
    'cfg5_sample': lambda: build_cache_sample('gpt2_cfg5_sample', 'gpt2', 5, 'rich', 32, lambda b: 64 + (b * 53) % 449, 2, [0, 9, 20, 31]),
    'cfg5_b64_sample': lambda: build_cache_sample('gpt2_cfg5_b64_sample', 'gpt2', 5, 'rich', 64, lambda b: 64 + (b * 53) % 449, 2, [0, 21, 42, 63]),
    'cfg5_b256_sample': lambda: build_cache_sample('gpt2_cfg5_b256_sample', 'gpt2', 5, 'rich', 256, lambda b: 64 + (b * 53) % 449, 2, [0, 85, 170, 255]),
    'cfg3_tail_sample': lambda: build_cache_sample('gpt2_cfg3_tail_sample', 'gpt2', 5, 'rich', 64, 1021, 3, [0, 21, 42, 63]),
    'xl1_sample': lambda: build_cache_sample('gpt2_xl1_sample', 'gpt2_xl', 0, 'baseline', 1, 300, 2, [0]),
    'tiny': lambda: build('tiny_b3', 'tiny', 3, 'rich', 3, 5, 12, set(range(17)), True, 1),
    'tiny3': lambda: build('tiny3_b2', 'tiny3', 4, 'rich', 2, 7, 20, set(range(27)), True, 1),
    'small_rich': lambda: build('gpt2_rich_b1', 'gpt2', 5, 'rich', 1, 6, 6, set(range(12)), False, 1),
    'cfg2': lambda: build('gpt2_cfg2', 'gpt2', 0, 'baseline', 8, 128, 256, spread(384, 128), False, 8),
    'xl': lambda: build('gpt2_xl_b1', 'gpt2_xl', 0, 'baseline', 1, 4, 4, set(range(8)), False, 1),
}

if __name__ == '__main__':
    for t in sys.argv[1:] or ['tiny', 'tiny3', 'small_rich']:
        TARGETS[t]()
