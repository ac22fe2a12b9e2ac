"""vesta.interp of the drop-in package (vesta/interp.py:92,233 in the reference: `parse`, `run`).

`parse` is this backend's own front end for the same grammar. `run`, the NumPy evaluator, is the reference's CPU
implementation: this backend has no CPU path of its own by design, so `run` forwards to an installed copy of the
reference package when there is one (oracle/make_ref.py puts it under oracle/_ref) and raises ImportError otherwise.
"""
import importlib.util
import os

from vesta_gpu_b200.syntax import parse    # noqa: F401

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'oracle', '_ref', 'vesta', 'interp.py')
_run = None


def run(text, residue):
    """evaluate a program on the CPU with the reference interpreter (residue: name -> ndarray or scalar; emits write
    into it) -> env: name -> (array, axes)"""
    global _run
    if _run is None:
        if not os.path.exists(_REF):
            raise ImportError('vesta.interp.run is the reference\'s NumPy interpreter; this GPU backend ships no CPU evaluator. '
                              'Install a copy of the reference package with `python oracle/make_ref.py <checkout>`.')
        spec = importlib.util.spec_from_file_location('vesta_reference_interp', _REF)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _run = mod.run
    return _run(text, residue)
