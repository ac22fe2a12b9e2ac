"""Shared helpers of the tests: golden fixtures and the comparison rules.

Tolerances (the parity rule of this backend): per-step logits within max-abs 2e-2 / relative 1e-2 of the
reference interpreter; greedy tokens identical wherever the reference top-1 margin exceeds 1e-2.
The measured differences are around 4e-4, so the tests also hold a tighter bound that would catch
a dropped bias or a wrong rounding point.
"""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
ABS_TOL, REL_TOL, MARGIN = 2e-2, 1e-2, 1e-2
TIGHT = 2e-3


def load(name):
    g = np.load(os.path.join(GOLDEN, name + '.npz'))
    return g


def close(got, ref):
    """the north-star rule: |got - ref| <= 2e-2 or <= 1e-2 * |ref|"""
    d = np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64))
    return bool(np.all((d <= ABS_TOL) | (d <= REL_TOL * np.abs(ref))))


def fixture_inputs(g):
    from vesta_gpu_b200.shapes import SHAPES
    sh = SHAPES[str(g['shape'])]
    prompts = g['prompts']
    return sh, int(g['seed']), str(g['init']), prompts, int(g['gen']), [int(v) for v in g['keep']], int(g['stride'])


def teacher_tokens(g, i, P):
    """token fed at every position of sequence i: the prompt, then the reference's own choices"""
    prompts = g['prompts']
    toks = g[f'tokens_{i}']
    steps = len(toks)
    return np.array([prompts[i, t] if t < P else toks[t - 1] for t in range(steps)], np.int32)
