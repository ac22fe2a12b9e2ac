"""Drop-in alias package: `from vesta.gpt2 import VestaGPT2`, `vesta.lower.lower`,
`vesta.launch.Kernel` resolve to the B200 backend (vesta_gpu_b200), under the module names of
the reference package (vesta/__init__.py:1-12). The NumPy interpreter of the reference
(vesta.interp) is its CPU oracle and has no counterpart here; only its parser does
(vesta_gpu_b200.syntax)."""
from vesta_gpu_b200 import PROGRAMS, __version__      # noqa: F401
