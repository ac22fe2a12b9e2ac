"""The decode-step program on the GPU: Hugging Face style weights as residue, lowered to one
persistent kernel per step.

    m = VestaGPT2(hf, dtype='f16', batch=8, tmax=1024)
    m.reset(); m.x.copy_(tok); m.t.fill_(p); m.step()     # one decode step
    m.logits(), m.next()                                    # views, no sync

Same surface as the reference binding (vesta/gpt2.py:18-55): `gpt2_weights`, and `VestaGPT2`
with `W, B, tmax, keys, vals, x, t, low, k, weight_bytes, reset, step, logits, next, kv_bytes`.
With feedback on, each step writes its chosen token into x and advances t, so generation is
back-to-back launches with nothing from the host in between. The sizes (layers, width, heads,
MLP width, vocabulary) are read from the weights instead of being fixed to GPT-2 small
(vesta/gpt2.py:16), so an XL-shaped model runs through the same code.
"""
import torch

from . import PROGRAMS
from .launch import Kernel, TORCH_DT
from .lower import lower
from .program_text import decode_program
from .shapes import Shape

E_HEAD = 64


def gpt2_weights(hf):
    """state_dict under Hugging Face names -> residues of the step program, per-layer tensors stacked on l"""
    sd = hf.state_dict()
    L = 0
    while f'transformer.h.{L}.ln_1.weight' in sd:
        L += 1
    st = lambda n: torch.stack([sd[f'transformer.h.{l}.{n}'] for l in range(L)])
    return dict(wte=sd['transformer.wte.weight'], wpe=sd['transformer.wpe.weight'],
                ln1w=st('ln_1.weight'), ln1b=st('ln_1.bias'), qkvw=st('attn.c_attn.weight'), qkvb=st('attn.c_attn.bias'),
                ow=st('attn.c_proj.weight'), ob=st('attn.c_proj.bias'), ln2w=st('ln_2.weight'), ln2b=st('ln_2.bias'),
                fcw=st('mlp.c_fc.weight'), fcb=st('mlp.c_fc.bias'), pw=st('mlp.c_proj.weight'), pb=st('mlp.c_proj.bias'),
                lnfw=sd['transformer.ln_f.weight'], lnfb=sd['transformer.ln_f.bias'])


def shape_of(W, heads=None):
    N, D = W['wte'].shape
    L, _, F = W['fcw'].shape
    H = heads or D // E_HEAD
    return Shape('model', L=L, D=D, H=H, E=D // H, F=F, N=N, C=W['wpe'].shape[0])


class VestaGPT2:
    def __init__(self, hf, dtype='f16', batch=1, tmax=1024, feedback=True, program=None, timing=False,
                 blocks_per_sm=None, per_sequence_t=False, device=None, prompt_len=0, slab_tiles=None, tune=None, without=()):
        """program: path of a .vst file; default: the step program for the sizes of the weights
        (identical to programs/gpt2.vst for GPT-2 small), `without` naming the shifts and biases it leaves out
        (program_text.ADDITIVE). Weights the program does not receive are not bound. per_sequence_t: every sequence keeps its
        own position t[b] (ragged batches); default one position for the whole batch as in the
        reference. prompt_len > 0 adds the buffers `prompt` (batch, prompt_len) and `plen` (batch,): the
        kernel then feeds prompt[b][t+1] while t + 1 < plen[b] and its own choice afterwards."""
        tdt = TORCH_DT[dtype]
        dev = torch.device('cuda', torch.cuda.current_device() if device is None else device)
        self.device = dev
        self.W = {k: v.detach().to(dev, tdt).contiguous() for k, v in gpt2_weights(hf).items()}
        self.shape = shape_of(self.W)
        sh = self.shape
        self.B, self.tmax = batch, tmax
        self.keys = torch.zeros(batch, sh.L, tmax, sh.H, sh.E, device=dev, dtype=tdt)
        self.vals = torch.zeros_like(self.keys)
        self.x = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.t = torch.zeros(batch if per_sequence_t else 1, dtype=torch.int32, device=dev)
        R = {'x': self.x, 't': self.t, **self.W, 'keys': self.keys, 'vals': self.vals}
        if prompt_len:
            self.prompt = torch.zeros(batch, prompt_len, dtype=torch.int32, device=dev)
            self.plen = torch.zeros(batch, dtype=torch.int32, device=dev)
        names = {torch.int32: 'i32', torch.float16: 'f16', torch.float32: 'f32'}
        spec = {n: (((batch,) if per_sequence_t else ()), 'i32') if n == 't' else (tuple(v.shape), names[v.dtype])
                for n, v in R.items() if n not in ('prompt', 'plen')}
        if program is None:
            text = decode_program(sh, without=tuple(without))
        else:
            text = open(program, encoding='utf-8').read()
        from .lower import recognise
        recv = set(recognise(text)[2])
        self.W = {n: v for n, v in self.W.items() if n in recv}
        R = {n: v for n, v in R.items() if n in recv}
        spec = {n: v for n, v in spec.items() if n in recv}
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        per_token = ('x', 'keys', 'vals') + (('t',) if per_sequence_t else ())
        self.low = lower(text, spec, axis_max={'s': tmax}, batch=batch, per_token=per_token,
                         outputs=('logit', 'next'), feedback={'x': 'next', 't': 1} if feedback else None,
                         timing=timing, grid=sms, prompt_len=prompt_len if feedback else 0, slab_tiles=slab_tiles, tune=tune)
        self._text, self._tune, self._prefill_engines = text, tune, {}
        self.k = Kernel(self.low, device=dev.index, blocks_per_sm=blocks_per_sm)
        if prompt_len and feedback:
            R = dict(R, prompt=self.prompt, plen=self.plen)
        self.k.bind(R)
        self.weight_bytes = sum(v.numel() * v.element_size() for n, v in self.W.items() if n != 'wpe') \
            + sh.D * self.W['wpe'].element_size()

    def reset(self):
        self.keys.zero_(); self.vals.zero_(); self.t.zero_()

    def step(self, steps=1):
        self.k.launch(steps)

    def step_host(self, tokens_host, next_host):
        """one step for a host-side loop: tokens_host (pinned int32 [batch]) becomes x, the chosen tokens (the
        `next` values, float32 [batch] as in the reference's scratch) land in next_host (pinned); returns when
        they have"""
        nv = self.__dict__.get('_next_view')
        if nv is None:
            nv = self._next_view = self.next()              # (a view of the scratch area: made once, a host loop calls this per step)
        self.k.step_host(self.x, tokens_host, nv, next_host)

    def prefill(self, tokens, lengths=None, rows=None):
        """consume whole prompts as dense passes: all prompt positions of all sequences are cut into launches of `rows`
        (sequence, position) rows (default 1024 from 1 K positions, 256 from 256, else 128) through the large-batch kernel: tensor-core
        contractions where the shape allows, every row's K and V written before any row attends, so a row sees the rows
        of its own sequence before it. On return the cache holds every prompt position, x the first generated token
        of every sequence and t its position (= its prompt length). tokens: int array (batch, P); lengths: (batch,) or
        None for P everywhere (lengths that differ need per_sequence_t=True).
        The reference feeds the prompt one position per step (bench/g0_bench.py:172-173); prefill_stepwise does the same
        on the device."""
        import numpy as np
        tokens = np.asarray(tokens)
        B, P = tokens.shape
        if B != self.B:
            raise ValueError('prefill needs one prompt per sequence of the batch')
        lens = np.full(B, P, np.int32) if lengths is None else np.asarray(lengths, np.int32)
        if lens.min() < 1 or lens.max() > P or lens.max() > self.tmax:
            raise ValueError('prompt lengths must lie in 1..P and fit the cache')
        if self.t.numel() == 1 and lens.min() != lens.max():
            raise ValueError('prompts of different lengths need per_sequence_t=True')
        total = int(lens.sum())
        rows = int(rows or (1024 if total >= 1024 else 256 if total >= 256 else 128))
        eng = self._prefill_engines.get(rows)
        if eng is None:
            eng = self._prefill_engines[rows] = _PrefillRows(self, rows)
        self.reset()
        first = eng.run(tokens, lens)
        self.x.copy_(first)
        self.t.copy_(torch.from_numpy(lens[:self.t.numel()].copy()))
        if hasattr(self, 'prompt'):
            buf = np.zeros(tuple(self.prompt.shape), np.int32)
            w = min(P, buf.shape[1])
            buf[:, :w] = tokens[:, :w]
            self.prompt.copy_(torch.from_numpy(buf)); self.plen.copy_(torch.from_numpy(np.minimum(lens, buf.shape[1]).astype(np.int32)))

    def prefill_stepwise(self, tokens, lengths=None):
        """consume whole prompts one position per step, fed on the device (needs prompt_len >= the longest prompt and
        per_sequence_t when the lengths differ): the prompts go to the device once, then the kernel feeds itself, several
        steps per launch, until every prompt has been read; sequences shorter than the longest start late (negative
        positions) so that all of them end together. On return x holds the first generated token of every sequence and
        t its position. tokens: int array (batch, P), lengths: (batch,) or None for P everywhere."""
        import numpy as np
        tokens = np.asarray(tokens)
        B, P = tokens.shape
        if not hasattr(self, 'prompt') or B != self.B or P > self.prompt.shape[1]:
            raise ValueError('prefill_stepwise needs a model built with prompt_len >= the prompt length and the same batch')
        lens = np.full(B, P, np.int32) if lengths is None else np.asarray(lengths, np.int32)
        if lens.min() < 1 or lens.max() > P:
            raise ValueError('prompt lengths must lie in 1..P')
        pmax = int(lens.max())
        if self.t.numel() == 1 and lens.min() != pmax:
            raise ValueError('prompts of different lengths need per_sequence_t=True')
        buf = np.zeros(tuple(self.prompt.shape), np.int32)
        buf[:, :P] = tokens
        self.reset()
        self.prompt.copy_(torch.from_numpy(buf)); self.plen.copy_(torch.from_numpy(lens))
        start = (lens - pmax).astype(np.int32)
        self.t.copy_(torch.from_numpy(start[:self.t.numel()]))
        self.x.copy_(torch.from_numpy(np.where(start == 0, tokens[:, 0], 0).astype(np.int32)))
        self.k.launch(pmax)

    def state(self):
        """the decode state (cache, tokens, positions) as CPU tensors, for load_state() on a model of the same
        shape, batch and tmax: generation then continues where it stood"""
        return {'keys': self.keys.cpu(), 'vals': self.vals.cpu(), 'x': self.x.cpu(), 't': self.t.cpu()}

    def load_state(self, st):
        for name in ('keys', 'vals', 'x', 't'):
            dst, src = getattr(self, name), st[name]
            if tuple(dst.shape) != tuple(src.shape) or dst.dtype != src.dtype:
                raise ValueError(f'state[{name!r}] is {tuple(src.shape)} {src.dtype}, the model holds {tuple(dst.shape)} {dst.dtype}')
            dst.copy_(src)

    def logits(self):
        return self.k.view('logit')

    def next(self):
        return self.k.view('next')

    def kv_bytes(self, n_ctx):
        sh = self.shape
        return 2 * sh.L * self.B * n_ctx * sh.D * self.keys.element_size()


class _PrefillRows:
    """The dense prompt pass behind VestaGPT2.prefill: a second lowering of the same program for `rows` rows of
    (cache sequence, position) that share the model's weights and caches (lower(..., row_seq=True))."""

    def __init__(self, model, rows):
        dev, sh = model.device, model.shape
        self.model, self.R = model, rows
        self.x = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.t = torch.full((rows,), -1, dtype=torch.int32, device=dev)
        self.seq = torch.zeros(rows, dtype=torch.int32, device=dev)
        R = {'x': self.x, 't': self.t, **model.W, 'keys': model.keys, 'vals': model.vals}
        names = {torch.int32: 'i32', torch.float16: 'f16', torch.float32: 'f32'}
        spec = {n: (tuple(v.shape), names[v.dtype]) for n, v in R.items()}
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        tune = dict(model._tune or {})
        tune.setdefault('ln_dist', True)            # rows normalised once on the grid: what the tensor-core contractions read
        self.low = lower(model._text, spec, axis_max={'s': model.tmax}, batch=rows, per_token=('x', 'keys', 'vals', 't'),
                         outputs=('logit', 'next'), feedback=None, grid=sms, row_seq=True, tune=tune)
        self.k = Kernel(self.low, device=dev.index)
        self.k.bind(dict(R, row_seq=self.seq))

    def run(self, tokens, lens):
        """tokens (B, P), lens (B,) numpy -> int32 tensor (B,) on the device: the token chosen after every prompt"""
        import numpy as np
        B, R = tokens.shape[0], self.R
        seqs = np.repeat(np.arange(B, dtype=np.int32), lens)
        pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
        tok = tokens[seqs, pos].astype(np.int32)
        first = torch.zeros(B, dtype=torch.int32, device=self.model.device)
        for i in range(0, len(seqs), R):
            n = min(R, len(seqs) - i)
            x, t, s = np.zeros(R, np.int32), np.full(R, -1, np.int32), np.zeros(R, np.int32)
            x[:n], t[:n], s[:n] = tok[i:i + n], pos[i:i + n], seqs[i:i + n]
            # Only the last position of a prompt needs logits: those rows go first (the order of the rows is free), all
            # others carry the kernel's "nobody reads these logits" mark, and the logits phase runs for the slabs of
            # 64 rows that hold an unmarked row (none, in most launches of a long prompt).
            want = np.zeros(R, bool)
            want[:n] = t[:n] == lens[s[:n]] - 1
            order = np.argsort(~want, kind='stable')
            x, t, s, want = x[order], t[order], s[order], want[order]
            self.x.copy_(torch.from_numpy(x)); self.t.copy_(torch.from_numpy(t))
            self.seq.copy_(torch.from_numpy(np.where(want, s, s | ROW_NO_LOGITS).astype(np.int32)))
            self.k.launch()
            last = np.flatnonzero(want)                                # rows that are the last position of their prompt
            if len(last):
                rows = torch.from_numpy(last).to(self.model.device)
                first[torch.from_numpy(s[last].astype(np.int64)).to(self.model.device)] = self.k.view('next')[rows].to(torch.int32)
        self.k.check()
        return first


ROW_NO_LOGITS = 0x40000000         # mark in row_seq (csrc/step_kernel.cuh): nobody reads the logits of this row
DEFAULT_PROGRAM = PROGRAMS / 'gpt2.vst'
