"""Model shapes of the decode-step family and the byte model of one step.

The byte model follows the reference's accounting (vesta/gpt2.py:44-45,54-55 and
bench/g0_bench.py:238-243): every weight element is read once per step (all residues
except the position table, of which one row is read) and every attended K and V element
is read once.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class Shape:
    name: str
    L: int      # layers
    D: int      # model width
    H: int      # heads
    E: int      # head width
    F: int      # MLP width
    N: int      # vocabulary
    C: int      # positions in the learned position table (n_ctx)

    @property
    def J(self):
        return 3 * self.D

    def weight_elems(self):
        """elements read per step: all weights once, one row of the position table"""
        L, D, F, N, J = self.L, self.D, self.F, self.N, self.J
        per_layer = 2 * D + D * J + J + D * D + D + 2 * D + D * F + F + F * D + D
        return N * D + L * per_layer + 2 * D + D

    def weight_bytes(self, elem=2):
        return self.weight_elems() * elem

    def kv_bytes_per_pos(self, elem=2):
        """K and V bytes one sequence reads per attended position, all layers"""
        return 2 * self.L * self.D * elem

    def step_bytes(self, ctx_lens, elem=2):
        """algorithmic bytes of one decode step: weights + KV of every sequence.
        ctx_lens: attended positions (t+1) per sequence."""
        return self.weight_bytes(elem) + self.kv_bytes_per_pos(elem) * int(sum(ctx_lens))


GPT2_SMALL = Shape('gpt2', L=12, D=768, H=12, E=64, F=3072, N=50257, C=1024)
GPT2_XL = Shape('gpt2_xl', L=48, D=1600, H=25, E=64, F=6400, N=50257, C=1024)
# small shapes for parity tests: same program family, everything a multiple of 16 except the vocabulary
TINY = Shape('tiny', L=2, D=128, H=2, E=64, F=256, N=211, C=64)
TINY3 = Shape('tiny3', L=3, D=192, H=3, E=64, F=320, N=333, C=96)

# twenty heads on two layers: at eight sequences more (sequence, head) pairs than SMs, so CTAs hold several attention items
HEADS20 = Shape('heads20', L=2, D=1280, H=20, E=64, F=512, N=517, C=48)

SHAPES = {s.name: s for s in (GPT2_SMALL, GPT2_XL, TINY, TINY3, HEADS20)}
