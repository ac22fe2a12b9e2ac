"""Alias of vesta_gpu_b200.lower under the reference module name."""
from vesta_gpu_b200.lower import *      # noqa: F401,F403
from vesta_gpu_b200 import lower as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
