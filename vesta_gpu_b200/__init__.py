"""B200-native backend for the Vesta GPT-2 decode step.

    vesta_gpu_b200.syntax    lexer/parser of the four-form language (law, fold, fork, residue)
    vesta_gpu_b200.lower     program -> placement plan for 148 SMs + CUDA source of one persistent kernel
    vesta_gpu_b200.launch    NVRTC compile and cooperative launch through the C ABI of libvesta_b200.so
    vesta_gpu_b200.gpt2      GPT-2 (any width/depth of the same step program) bound to that kernel
    vesta_gpu_b200.shard     batch partition of independent sequences over GPUs

The public names mirror the reference package `vesta` (vesta/__init__.py:1-12): the same
programs and the same lower / launch / gpt2 calls drive this backend.
"""
from pathlib import Path

__version__ = '0.1.0'
PROGRAMS = Path(__file__).resolve().parent / 'programs'
