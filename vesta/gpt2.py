"""Alias of vesta_gpu_b200.gpt2 under the reference module name."""
from vesta_gpu_b200.gpt2 import *      # noqa: F401,F403
from vesta_gpu_b200 import gpt2 as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
