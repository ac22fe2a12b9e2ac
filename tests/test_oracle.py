"""The CPU oracle (oracle/gpt2_numpy.py) against outputs of the reference interpreter itself
(tests/golden/*.npz, produced by tests/golden/make_golden.py from vesta.interp.run)."""
import numpy as np
import pytest

from oracle import gpt2_numpy as O
from vesta_gpu_b200.synth import make_weights
from helpers import load, fixture_inputs, close, TIGHT, MARGIN

_W = {}


def weights(sh, seed, init):
    key = (sh.name, seed, init)
    if key not in _W:
        _W.clear()                      # one model at a time: the XL weights take 6 GB as float32
        _W[key] = O.upcast(make_weights(sh, seed, init))
    return _W[key]


def check_fixture(name, seqs=None, steps=None):
    g = load(name)
    sh, seed, init, prompts, gen, keep, stride = fixture_inputs(g)
    W = weights(sh, seed, init)
    P = prompts.shape[1]
    for i in (range(prompts.shape[0]) if seqs is None else seqs):
        toks, margins = g[f'tokens_{i}'], g[f'margins_{i}']
        n = len(toks) if steps is None else steps
        r = O.decode(sh, W, prompts[i], n - P, keep_logits=set(keep), force=toks[P - 1:])
        sure = margins[:n] > MARGIN
        assert np.array_equal(r['tokens'][sure], toks[:n][sure]), name
        assert np.allclose(r['margins'], margins[:n], atol=TIGHT)
        for k, t in enumerate(keep):
            if t < n:
                assert close(r['logits'][t][::stride], g[f'logits_{i}'][k])
                assert np.abs(r['logits'][t][::stride] - g[f'logits_{i}'][k]).max() < TIGHT
                # the five best entries: same values at the reference's indices
                assert np.abs(r['logits'][t][g[f'top_idx_{i}'][k]] - g[f'top_val_{i}'][k]).max() < TIGHT


def check_samples(name):
    """sampled sequences of a large batch, two teacher-forced steps on seeded caches (the reference interpreter needs
    a second per position, so these fixtures start from a filled cache instead of a long prompt)"""
    from vesta_gpu_b200.shapes import SHAPES
    from vesta_gpu_b200.synth import make_cache
    g = load(name)
    sh, steps, stride = SHAPES[str(g['shape'])], int(g['steps']), int(g['stride'])
    W = weights(sh, int(g['seed']), str(g['init']))
    for i, b in enumerate(g['sample']):
        ctx = int(g['ctxs'][b])
        k0, v0 = make_cache(sh, int(g['cache_seed_base']) + int(b), ctx)
        keys = np.zeros((sh.L, ctx + steps, sh.H, sh.E), np.float16); vals = np.zeros_like(keys)
        keys[:, :ctx] = k0; vals[:, :ctx] = v0
        for s_ in range(steps):
            logit, nxt = O.step(sh, W, keys, vals, int(g[f'fed_{i}'][s_]), ctx + s_)
            assert np.abs(logit[::stride] - g[f'logits_{i}'][s_]).max() < TIGHT
            assert np.abs(logit[g[f'top_idx_{i}'][s_]] - g[f'top_val_{i}'][s_]).max() < TIGHT
            if g[f'margins_{i}'][s_] > MARGIN:
                assert nxt == int(g[f'tokens_{i}'][s_])


def test_tiny_all_steps():
    check_fixture('tiny_b3')


def test_tiny3_vocab_not_multiple_of_16():
    check_fixture('tiny3_b2')


def test_gpt2_small_rich_init():
    """non-zero biases and LayerNorm parameters"""
    check_fixture('gpt2_rich_b1')


def test_gpt2_small_first_steps_of_batch8():
    check_fixture('gpt2_cfg2', seqs=range(8), steps=4)


def test_gpt2_small_full_decode_sequence0():
    """batch-1 configuration: 128-token prompt + 256 greedy steps, every token and every kept logit row"""
    check_fixture('gpt2_cfg2', seqs=[0])


def test_gpt2_xl_shape():
    check_fixture('gpt2_xl_b1')


def test_gpt2_xl_batch16_sample():
    """two of 16 sequences of the XL shape at context 300 (runs next to the other XL test: the weights are shared)"""
    check_samples('gpt2_xl16_sample')


def test_gpt2_xl_batch1_sample():
    """the XL shape at batch 1, context 300"""
    check_samples('gpt2_xl1_sample')


def test_tie_goes_to_lowest_index():
    """gpt2.vst:81-82: next = min index whose logit equals the maximum"""
    logit = np.array([0.5, 2.0, 2.0, 1.0], np.float32)
    assert int(np.flatnonzero(logit == logit.max())[0]) == 1
    assert O.margin(logit) == 0.0


def test_kv_cache_rounds_to_fp16():
    """the emit rounds K and V to the cache dtype and the same step reads the rounded row back"""
    from vesta_gpu_b200.shapes import TINY
    W = weights(TINY, 3, 'rich')
    k16, v16 = O.new_cache(TINY, 4, np.float16)
    k32, v32 = O.new_cache(TINY, 4, np.float32)
    a, _ = O.step(TINY, W, k16, v16, 5, 0)
    b, _ = O.step(TINY, W, k32, v32, 5, 0)
    assert k16.dtype == np.float16 and np.array_equal(k16[0, 0], k32[0, 0].astype(np.float16))   # layer 0 sees the same input
    assert np.abs(a - b).max() < 1e-2 and not np.array_equal(a, b)


@pytest.mark.parametrize('name', ['gpt2_cfg3_sample', 'gpt2_cfg5_sample', 'gpt2_cfg5_b64_sample', 'gpt2_cfg5_b256_sample', 'gpt2_cfg3_tail_sample'])
def test_gpt2_small_deep_context_samples(name):
    """the batch-64 config at context 600 and at the last positions of a 1024-row cache (1021..1023), ragged batches of
    32, 64 and 256 with contexts 64..512"""
    check_samples(name)


def test_program_without_additive_parameters_in_the_reference_interpreter():
    """the statements without their shift / bias term, as vesta_gpu_b200 accepts them, evaluated by the reference
    interpreter itself (when a copy of the reference is installed): the same logits as the oracle computes with
    those parameters set to zero, which is what the GPU tests compare the kernel with"""
    import os
    from vesta_gpu_b200.program_text import decode_program, ADDITIVE
    from vesta_gpu_b200.shapes import TINY
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(here, 'oracle', '_ref', 'vesta', 'interp.py')):
        pytest.skip('no copy of the reference installed (python oracle/make_ref.py <checkout>)')
    from vesta.interp import run
    raw = make_weights(TINY, 5, 'rich')
    for without in (('qkvb', 'fcb'), ADDITIVE):
        text = decode_program(TINY, without=without)
        Wz = O.upcast({k: (np.zeros_like(v) if k in without else v) for k, v in raw.items()})
        Wr = {k: v for k, v in O.upcast(raw).items() if k not in without}
        keys, vals = O.new_cache(TINY, 4)
        rk, rv = O.new_cache(TINY, 4)
        for t, x in enumerate((7, 100, 3)):
            ref, _ = O.step(TINY, Wz, keys, vals, x, t)
            env = run(text, dict(Wr, x=x, t=t, keys=rk, vals=rv))
            assert np.abs(np.asarray(env['logit'][0]) - ref).max() < 1e-5, (without, t)
