"""Alias of vesta_gpu_b200.launch under the reference module name."""
from vesta_gpu_b200.launch import *      # noqa: F401,F403
from vesta_gpu_b200 import launch as _m

globals().update({k: v for k, v in vars(_m).items() if not k.startswith("__")})
