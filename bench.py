"""Decode throughput of the Vesta GPT-2 step on B200, one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

A step is one decode step of one batch. Protocol of the reference benchmark (bench/g0_bench.py:166-180): reset,
feed the prompt one token per step (untimed), then time K generation steps that run back to back with the kernel
feeding its own token; the median of --repeats runs is reported. The prompt is a seeded uniform token sequence and
the weights are seeded random-init fp16 (the pretrained checkpoint and prompt need a download).

Workloads: cfg1 = GPT-2 small batch 1, cfg2 = batch 8 (the default: the configuration the metric is quoted on), both
128-token prompts + 256 steps; cfg3 = batch 64 with 512-token prompts; xl1 / xl16 = XL shape at batch 1 / 16; cfg5 =
256 ragged sequences split over the GPUs. With --gpus N > 1 every rank (one process per GPU, torchrun) runs its own
sequences with no exchange on the step path; generated tokens are gathered to rank 0 at the end.

The line of the default run (cfg2) carries, beside the contract's keys:
`value`       tokens/s with everything resident in HBM (CUDA events around the K steps)
`e2e`         tokens/s through the public API with host buffers: every step copies the input tokens from pinned host
              memory, launches, and reads the chosen tokens back
`roofline`    algorithmic bytes per launch (all weights + attended K/V, the reference's byte model,
              vesta/gpt2.py:44-45,54-55) / mean launch duration, against the measured copy bandwidth
`prefill`     the prompt as dense passes of (sequence, position) rows against one position per step (both untimed in `value`)
`secondary`   the same measurements for cfg1 (batch 1), taken in the same run
`strong`      cfg5 (256 ragged sequences split evenly over the N GPUs): tokens/s, us per step and the fraction of the
              byte-model speed-up over one GPU
`ref_kernel`  the reference's own generated kernel (NVRTC, its stock VestaGPT2.step path) timed with the same protocol
              on the same GPU at batch 1 and 8, when a copy of the reference package is installed under oracle/_ref
`cpu_baseline` the reference interpreter (vesta/interp.py, `kind: reference`) on the host cores when oracle/_ref holds
              it, else the NumPy oracle (`kind: port`)
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np      # noqa: E402

WORKLOADS = {
    'cfg1': dict(shape='gpt2', batch=1, prompt=128, gen=256),
    'cfg2': dict(shape='gpt2', batch=8, prompt=128, gen=256),
    'cfg3': dict(shape='gpt2', batch=64, prompt=512, gen=512),
    'xl1': dict(shape='gpt2_xl', batch=1, prompt=128, gen=256),
    'xl16': dict(shape='gpt2_xl', batch=16, prompt=128, gen=256),
    # 256 sequences over all GPUs (strong scaling), ragged prompts of 64..512 tokens, per-sequence positions
    'cfg5': dict(shape='gpt2', batch=256, prompt=512, gen=256, ragged=(64, 512), total=True),
    'tiny': dict(shape='tiny3', batch=2, prompt=8, gen=16),
}
METRIC, UNIT = 'decode tokens/s', 'tokens/s'
REF_DIR = os.path.join(ROOT, 'oracle', '_ref')          # an installed copy of the reference package (oracle/make_ref.py)
# DRAM bytes (read + write) of one decode step from the ncu captures summarised under profiles/, each taken at the given
# context (attended positions per sequence). A bench launch attends more positions: the K/V part is scaled by the
# positions, the weights are read once either way. Workloads without a capture report null.
NCU_CAPTURE = {
    'cfg2': dict(bytes=291.0e6, positions=131.5, source='scaled from the ncu capture in profiles/vesta_step_gpt2_small_b1_b8.md (two steps at contexts 131 and 132) by the K/V bytes of this run\'s contexts'),
    'cfg1': dict(bytes=256.3e6, positions=131.5, source='scaled from the ncu capture in profiles/vesta_step_gpt2_small_b1_b8.md (two steps at contexts 131 and 132) by the K/V bytes of this run\'s contexts'),
    'cfg3': dict(bytes=1484.9e6, positions=513.5, source='scaled from the ncu capture in profiles/vesta_step_gpt2_small_b64.md (two steps at contexts 513 and 514) by the K/V bytes of this run\'s contexts'),
}
NCU_SOURCE = 'no capture of this workload for the current kernel: see profiles/'


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        return float(json.load(open(p))['hbm_gbs']), 'measured (MEASURED_PEAKS.json hbm_gbs, copy)'
    return 6650.0, 'fallback (earlier measurement on this pool)'


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs"""
    Q = 'clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,' \
        'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap'

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={index}', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '50'], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([v.strip() for v in line.split(',')])

    def mark(self):
        return len(self.rows)

    def summary(self, start=0, end=None):
        rows = [r for r in self.rows[start:end] if len(r) >= 7 and r[0].isdigit()] or \
               [r for r in self.rows if len(r) >= 7 and r[0].isdigit()]
        if not rows:
            return None
        sm = sorted(int(r[0]) for r in rows)
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = sorted({n for r in rows for n, v in zip(names, r[3:7]) if v.lower().startswith('active')})
        return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=int(rows[0][1]), reasons=reasons, samples=len(rows))

    def stop(self):
        if self.proc:
            time.sleep(0.12)
            self.proc.terminate()


def host_threads():
    """let NumPy's BLAS use every host core (torchrun exports OMP_NUM_THREADS=1); -> the threads it then runs on"""
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=os.cpu_count())
        n = [int(i.get('num_threads', 1)) for i in threadpool_info()]
        return max(n) if n else 1
    except Exception:
        return 1


# ------------------------------------------------------------------ the CPU arms
def reference_interpreter():
    """vesta.interp.run of the installed reference copy, loaded by file so that it cannot be confused with this
    repository's own `vesta` package; None when no copy is installed"""
    path = os.path.join(REF_DIR, 'vesta', 'interp.py')
    if not os.path.exists(path):
        return None
    spec = importlib.util.spec_from_file_location('vesta_reference_interp', path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.run


def cpu_steps(sh, weights16, t0, steps, warm=1, max_seconds=None, prefer_reference=True):
    """decode steps of ONE sequence on the host cores at positions t0, t0 + 1, ... (the cache before t0 is filled with
    random fp16 values: the time does not depend on them). The reference interpreter when a copy is installed, else
    the NumPy oracle. -> dict(kind, steps_per_second, seconds, steps)"""
    from oracle import gpt2_numpy as O
    from vesta_gpu_b200.program_text import decode_program
    run = reference_interpreter() if prefer_reference else None
    rng = np.random.default_rng(0)
    room = min(t0 + steps + warm + 1, sh.C)
    keys = (rng.standard_normal((sh.L, room, sh.H, sh.E), dtype=np.float32) * 0.1).astype(np.float16)
    vals = keys.copy()
    W = O.upcast(weights16)
    text = decode_program(sh)

    def one(x, t):
        t = min(t, room - 1)
        if run is None:
            return O.step(sh, W, keys, vals, x, t)[1]
        return int(run(text, dict(W, x=int(x), t=int(t), keys=keys, vals=vals))['next'][0])
    x = 1
    for _ in range(warm):
        x = one(x, t0)
    start = time.perf_counter()
    done = 0
    for i in range(steps):
        x = one(x, t0 + i)
        done += 1
        if max_seconds and time.perf_counter() - start > max_seconds:
            break
    dt = time.perf_counter() - start
    return dict(kind='port' if run is None else 'reference', steps_per_second=done / dt, seconds=dt, steps=done)


def _cpu_worker(job):
    """one host process: decode steps of one sequence (top-level so that multiprocessing can start it)"""
    shape, t0, steps, max_seconds, threads = job
    os.environ['OMP_NUM_THREADS'] = str(threads)
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=threads)
    except Exception:
        pass
    from vesta_gpu_b200.shapes import SHAPES
    from vesta_gpu_b200.synth import make_weights
    sh = SHAPES[shape]
    return cpu_steps(sh, make_weights(sh, 0), t0, steps, warm=1, max_seconds=max_seconds)


def cpu_steps_all_cores(sh, batch, t0, steps, max_seconds):
    """The CPU implementation on all the host cores it can use: the interpreter runs one sequence at a time and is
    bound by NumPy gathers, so min(batch, cores) sequences of the batch run side by side, one process each (fewer for
    the XL shape, whose fp32 weights take 6 GB per process). -> dict(kind, value = sequence-steps per second over all
    processes, processes, threads, steps, seconds)"""
    import multiprocessing as mp
    cores = os.cpu_count() or 1
    nproc = max(1, min(batch, cores, 2 if sh.weight_bytes() > (1 << 30) else cores))
    threads = max(1, cores // nproc)
    if nproc == 1:
        res = [_cpu_worker((sh.name, t0, steps, max_seconds, threads))]
    else:
        with mp.get_context('spawn').Pool(nproc) as pool:
            res = pool.map(_cpu_worker, [(sh.name, t0, steps, max_seconds, threads)] * nproc)
    secs = max(r['seconds'] for r in res)
    done = min(r['steps'] for r in res)
    return dict(kind=res[0]['kind'], value=sum(r['steps'] for r in res) / secs, processes=nproc, threads=nproc * threads, steps=done, seconds=secs)


def cpu_sample_text(r, wl, P):
    how = 'vesta/interp.py of the installed reference copy' if r['kind'] == 'reference' else 'NumPy port of the interpreter (no reference copy under oracle/_ref)'
    return (f'{r["steps"]} consecutive decode steps at positions {P}..{P + r["steps"] - 1} of {r["processes"]} of the {wl["batch"]} sequences, '
            f'one process per sequence side by side ({r["seconds"]:.1f} s), {how}')


def run_reference(args, wl, sh):
    """the reference arm: the reference's own CPU implementation of the path (vesta/interp.py from the installed copy;
    the NumPy port of its arithmetic when there is none) on the host cores, rank 0 only. A step is one decode step of
    the sampled sequences, at the positions the GPU arm's timed steps run at."""
    if int(os.environ.get('RANK', '0')) != 0:
        return
    P, K = wl['prompt'], max(1, args.steps)
    r = cpu_steps_all_cores(sh, wl['batch'], P, K, max_seconds=150)
    tps = r['value']
    line = dict(metric=METRIC, value=tps, unit=UNIT, impl='reference', n_gpus=args.gpus, steps=r['steps'], warmup=1,
                ms_per_step=1e3 * r['seconds'] / r['steps'], higher_is_better=True, scaling='weak', vs_baseline=None,
                dtype='f32 accumulate over fp16-rounded weights', data='synthetic',
                config=dict(workload=args.workload, **{k: v for k, v in wl.items() if k != 'total'}, contexts=[P + 1, P + r['steps']]),
                cpu_baseline=dict(value=tps, unit=UNIT, cores=r['threads'], kind=r['kind'], sample=cpu_sample_text(r, wl, P)),
                e2e=dict(value=tps, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ------------------------------------------------------------------ the reference's own GPU kernel
def run_ref_kernel(args, wl, sh):
    """(internal: a subprocess of the default run) the reference package's own kernel through its stock
    VestaGPT2(...).step() path, protocol of bench/g0_bench.py:166-180; prints one JSON object"""
    sys.path.insert(0, REF_DIR)                      # before this repository's own `vesta`
    import torch
    from vesta.gpt2 import VestaGPT2 as RefGPT2       # the reference's, from the installed copy
    from vesta_gpu_b200.synth import SynthGPT2, make_prompts
    B, P, K = wl['batch'], wl['prompt'], args.steps
    v = RefGPT2(SynthGPT2(sh, seed=0), batch=B, tmax=P + K + 1)
    prompt = torch.from_numpy(make_prompts(sh, B, P, seed=1).copy()).cuda()
    times, toks0 = [], None
    for r in range(args.repeats + 1):                # the first pass is the warm-up
        v.reset()
        for i in range(P):
            v.x.copy_(prompt[:, i]); v.step()
        toks = [v.x.clone()]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            v.step(); toks.append(v.x.clone())
        e1.record()
        torch.cuda.synchronize()
        if r:
            times.append(e0.elapsed_time(e1) * 1e-3)
        toks0 = torch.stack(toks[:K], 1).cpu().numpy()
    med = statistics.median(times)
    print(json.dumps(dict(batch=B, steps=K, ms_per_step=1e3 * med / K, tokens_per_s=B * K / med, grid=int(v.k.grid), block=int(v.k.block),
                          barriers_per_step=int(v.low.barriers_per_launch), tokens=toks0[:, :32].tolist())))


def ref_kernel_block(args, ours_tokens):
    """time the reference's own kernel at batch 1 and 8 in child processes; -> dict for the JSON line"""
    if not os.path.exists(os.path.join(REF_DIR, 'vesta', 'lower.py')):
        return dict(unavailable='no copy of the reference package under oracle/_ref (oracle/make_ref.py installs one)')
    out = {}
    for name in ('cfg1', 'cfg2'):
        cmd = [sys.executable, os.path.abspath(__file__), '--impl', 'ref-kernel', '--workload', name, '--steps', str(args.steps),
               '--repeats', str(min(args.repeats, 3))]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
            line = [l for l in r.stdout.splitlines() if l.startswith('{')]
            if r.returncode != 0 or not line:
                out[name] = dict(failed=(r.stderr or r.stdout).strip().splitlines()[-1][:200] if (r.stderr or r.stdout).strip() else f'exit {r.returncode}')
                continue
            d = json.loads(line[-1])
            toks = d.pop('tokens')
            if name in ours_tokens:
                n = min(len(toks[0]), ours_tokens[name].shape[1])
                d['first_tokens_equal_ours'] = round(float((np.array(toks)[:, :n] == ours_tokens[name][:, :n]).mean()), 4)
            out[name] = d
        except subprocess.TimeoutExpired:
            out[name] = dict(failed='no result within 240 s')
    out['how'] = 'the reference package (installed copy) lowered and JIT-compiled by its own vesta/lower.py + vesta/launch.py for this GPU, one launch per step'
    return out


# ------------------------------------------------------------------ our arm
class Run:
    """one workload on this rank's GPU: model, prompts and the timed loops"""

    def __init__(self, name, args, rank, world, local):
        import torch
        from vesta_gpu_b200.shapes import SHAPES
        from vesta_gpu_b200.synth import SynthGPT2, make_prompts
        from vesta_gpu_b200.gpt2 import VestaGPT2
        self.torch, self.name, self.args, self.rank, self.world = torch, name, args, rank, world
        wl = self.wl = dict(WORKLOADS[name])
        sh = self.sh = SHAPES[wl['shape']]
        P, K, Wm = wl['prompt'], args.steps, max(args.warmup, 3)
        self.P, self.K, self.Wm = P, K, Wm
        self.total = bool(wl.get('total'))
        if self.total and wl['batch'] % world:
            raise SystemExit(f'{wl["batch"]} sequences do not split over {world} GPUs')
        B = self.B = wl['batch'] // world if self.total else wl['batch']
        tmax = P + max(K, Wm) + 1
        if tmax > sh.C:
            raise SystemExit(f'prompt + steps = {tmax} exceeds the position table ({sh.C})')
        self.hf = SynthGPT2(sh, seed=0)
        self.ragged = wl.get('ragged')
        if self.ragged:
            from vesta_gpu_b200.synth import make_ragged_prompts
            from vesta_gpu_b200.shard import partition
            lens_all, toks_all = make_ragged_prompts(sh, B * world, self.ragged[0], self.ragged[1], seed=1)
            self.mine = partition(lens_all, world)[rank]
            lens, prompts = lens_all[self.mine], toks_all[self.mine]
            m = VestaGPT2(self.hf, batch=B, tmax=tmax, device=local, per_sequence_t=True, prompt_len=P)
            m.prompt.copy_(torch.from_numpy(prompts[:, :P].copy()))
            m.plen.copy_(torch.from_numpy(lens))
            self.start = torch.from_numpy((lens - P).astype(np.int32)).cuda()         # <= 0: every prompt ends at step P
            self.first_tok = torch.from_numpy(np.where(lens == P, prompts[:, 0], 0).astype(np.int32)).cuda()
            self.ctx_lens = [[int(n) + i + 1 for n in lens_all] for i in range(K)]    # attended positions of every sequence per step
            self.mine_lens = lens
        else:
            self.mine = list(range(rank * B, (rank + 1) * B))
            prompts = make_prompts(sh, B * world, P, seed=1)[rank * B:(rank + 1) * B]      # every rank its own sequences
            m = VestaGPT2(self.hf, batch=B, tmax=tmax, device=local)
            self.pd = torch.from_numpy(prompts.copy()).cuda()
            self.ctx_lens = [[P + i + 1] * (B * world) for i in range(K)]
        self.m = m

    def prefill(self):
        m = self.m
        m.reset()
        if self.ragged:
            # the kernel feeds itself from the prompt buffer; sequences start late so that all prompts end together
            m.t.copy_(self.start); m.x.copy_(self.first_tok)
            m.step(self.P)
        else:
            for t in range(self.P):
                m.x.copy_(self.pd[:, t])
                m.step()

    def sync_all(self):
        torch = self.torch
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    def device_loop(self, repeats):
        """-> seconds of the K timed steps per repeat (CUDA events; the kernel feeds x and t itself)"""
        torch, m = self.torch, self.m
        self.prefill(); m.step(self.Wm); torch.cuda.synchronize(); m.k.check()          # warm-up: prompt + Wm steps, untimed
        times = []
        for _ in range(repeats):
            self.prefill()
            self.sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            m.k.launch(self.K, per_launch=self.args.per_launch)
            e1.record()
            self.sync_all()
            times.append(e0.elapsed_time(e1) * 1e-3)
        m.k.check()
        return times

    def token_stream(self):
        """the generated tokens, stepwise (untimed): [B, K] on the device"""
        torch, m = self.torch, self.m
        self.prefill()
        stream = [m.x.clone()]
        for _ in range(self.K - 1):
            m.step(); stream.append(m.x.clone())
        torch.cuda.synchronize()
        return torch.stack(stream, 1)

    def host_loop(self, repeats, stream):
        """end to end: host buffers every step. -> (seconds per repeat, fraction of tokens equal to the device loop's)"""
        torch, m, B, K = self.torch, self.m, self.B, self.K
        hx = torch.empty(B, dtype=torch.int32).pin_memory()
        hn = torch.empty(B, dtype=torch.float32).pin_memory()
        times, seen = [], []
        for _ in range(repeats):
            self.prefill()
            hx.copy_(m.x.cpu())
            self.sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            seen = []
            hxn, hnn = hx.numpy(), hn.numpy()                # the same pinned buffers, seen from numpy (cheaper per-step host work)
            for _ in range(K):
                # host -> device: this step's input tokens; one launch; device -> host: the chosen tokens; synchronise
                m.step_host(hx, hn)
                hxn[:] = hnn                                 # the chosen tokens (float32 in the scratch, as in the reference) are the next input
                seen.append(torch.from_numpy(hxn.copy()))
            e1.record()
            self.sync_all()
            times.append(e0.elapsed_time(e1) * 1e-3)
        # after K host-driven steps hx holds the token chosen by step K; the device loop's stream holds the tokens before
        # steps 1..K. fp32 atomics make the last bits, and hence near-ties over hundreds of free-running steps, run-dependent
        same = round(float((torch.stack(seen[:-1], 1) == stream[:, 1:].cpu()).float().mean()), 4) if K > 1 else None
        return times, same

    def prefill_block(self):
        """the prompt as dense passes (VestaGPT2.prefill: rows of (sequence, position), tensor-core contractions) against
        the reference's protocol of one position per step; -> dict or None (ragged workloads feed prompts on the device)"""
        if self.ragged:
            return None
        torch, m = self.torch, self.m
        prompts = self.pd.cpu().numpy()

        def timed(fn, n=3):
            out = []
            for _ in range(n):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record()
                torch.cuda.synchronize()
                out.append(e0.elapsed_time(e1))
            return statistics.median(out)
        m.prefill(prompts); torch.cuda.synchronize()              # builds the second lowering and its weight image, untimed
        dense = timed(lambda: m.prefill(prompts))
        first_dense = m.x.clone()
        step = timed(self.prefill)
        rows = max(m._prefill_engines)
        return dict(positions=int(prompts.size), dense_ms=dense, one_position_per_step_ms=step, rows_per_launch=rows,
                    tensor_core_contractions=bool(m._prefill_engines[rows].low.dims['tcl']),
                    first_tokens_equal=round(float((first_dense == m.x).float().mean()), 4))

    def bytes_per_step(self):
        """algorithmic bytes of one step on one GPU: every weight once + the attended K/V of its sequences"""
        return sum(self.sh.weight_bytes() + self.sh.kv_bytes_per_pos() * sum(c) / self.world for c in self.ctx_lens) / self.K

    def reduce_max(self, *vals):
        if self.world == 1:
            return vals
        import torch.distributed as dist
        tt = self.torch.tensor(list(vals), device='cuda', dtype=self.torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return tuple(float(v) for v in tt)

    def measure(self, repeats, with_e2e=True):
        """-> (dict of the measured figures, token stream on the device)"""
        times = self.device_loop(repeats)
        stream = self.token_stream()
        med = statistics.median(times)
        out = dict(cv=round(statistics.pstdev(times) / statistics.mean(times), 4))
        e2e_med, same = None, None
        if with_e2e:
            e2e_times, same = self.host_loop(max(1, min(3, repeats)), stream)
            e2e_med = statistics.median(e2e_times)
        med, e2e_med = self.reduce_max(med, e2e_med or 0.0)
        B, K, world = self.B, self.K, self.world
        peak, peak_src = peaks()
        bps = self.bytes_per_step()
        achieved = bps / (med / K) / 1e9
        spl = min(self.args.per_launch, K)
        cap = NCU_CAPTURE.get(self.name) if world == 1 else None
        traffic = None
        if cap:
            mean_pos = sum(sum(c) for c in self.ctx_lens) / K / (B * world)
            traffic = (cap['bytes'] + B * (mean_pos - cap['positions']) * self.sh.kv_bytes_per_pos()) * spl
        out.update(value=B * world * K / med, ms_per_step=1e3 * med / K,
                   contexts=[min(self.ctx_lens[0]), max(self.ctx_lens[-1])],
                   roofline=dict(bound='hbm', achieved=achieved, peak=peak, unit='GB/s', frac=achieved / peak, traffic=traffic,
                                 traffic_source=(cap['source'] if cap else NCU_SOURCE),
                                 peak_source=peak_src, bytes_per_step=bps, bytes_per_launch=bps * spl, kernel='vesta_step',
                                 frac_of_8tbs=achieved / 8000.0),
                   gpu_launches=-(-K // self.args.per_launch))
        if with_e2e:
            out['e2e'] = dict(value=B * world * K / e2e_med, unit=UNIT, h2d_bytes_per_step=B * 4, d2h_bytes_per_step=B * 4,
                              tokens_match_device_loop=same)
        return out, stream


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=256)
    ap.add_argument('--warmup', type=int, default=8)
    ap.add_argument('--repeats', type=int, default=5)
    ap.add_argument('--per-launch', type=int, default=16, help='decode steps inside one kernel launch (1: a launch per step)')
    ap.add_argument('--workload', default='cfg2', choices=sorted(WORKLOADS))
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'ref-kernel'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='only the headline workload: no secondary, strong or ref_kernel blocks')
    args = ap.parse_args()
    from vesta_gpu_b200.shapes import SHAPES
    wl = dict(WORKLOADS[args.workload])
    sh = SHAPES[wl['shape']]
    if args.impl == 'reference':
        return run_reference(args, wl, sh)
    if args.impl == 'ref-kernel':
        return run_ref_kernel(args, wl, sh)

    import torch
    import torch.distributed as dist
    from vesta_gpu_b200.shard import gather_tokens

    rank, world = int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} needs {args.gpus} ranks (torchrun --nproc-per-node {args.gpus}); WORLD_SIZE is {world}')
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))

    sampler = ClockSampler(local) if rank == 0 else None
    run = Run(args.workload, args, rank, world, local)
    mark0 = sampler.mark() if sampler else 0
    res, stream = run.measure(args.repeats)
    mark1 = sampler.mark() if sampler else 0
    prefill = run.prefill_block() if (world == 1 and not args.no_extras) else None
    all_tokens = gather_tokens(stream.to(torch.int32), list(run.mine), run.B * world)
    if rank == 0:
        assert all_tokens.shape == (run.B * world, run.K)
    ours_tokens = {args.workload: stream.cpu().numpy()} if world == 1 else {}
    total, B, K = run.total, run.B, run.K
    del run

    extras = not args.no_extras and args.workload == 'cfg2'
    secondary, strong = None, None
    if extras and world == 1:
        r1 = Run('cfg1', args, rank, world, local)
        s1, st1 = r1.measure(min(args.repeats, 3))
        ours_tokens['cfg1'] = st1.cpu().numpy()
        secondary = dict(cfg1=dict(workload='cfg1', **{k: v for k, v in WORKLOADS['cfg1'].items()}, unit=UNIT, **s1))
        del r1
    if extras:
        # the batch-sharded configuration: 256 ragged sequences, 256 / N per GPU, no exchange on the step path
        r5 = Run('cfg5', args, rank, world, local)
        s5, st5 = r5.measure(min(args.repeats, 3), with_e2e=False)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g5 = gather_tokens(st5.to(torch.int32), list(r5.mine), r5.B * world)
        e1.record(); torch.cuda.synchronize()
        gather_ms = e0.elapsed_time(e1)
        if rank == 0:
            assert g5.shape == (256, r5.K)
            W, kv = r5.sh.weight_bytes(), r5.sh.kv_bytes_per_pos() * sum(sum(c) for c in r5.ctx_lens) / r5.K      # KV bytes of all 256 sequences per step
            ideal = (W + kv) / (W + kv / world)               # every GPU still streams all the weights per step
            strong = dict(workload='cfg5', sequences=256, sequences_per_gpu=r5.B, value=s5['value'], unit=UNIT, ms_per_step=s5['ms_per_step'],
                          contexts=s5['contexts'], roofline_frac=s5['roofline']['frac'], cv=s5['cv'],
                          byte_model_speedup_over_one_gpu=round(ideal, 3), gather_ms=round(gather_ms, 3),
                          note='speed-up over one GPU = value / (the value of the --gpus 1 run); the byte model W + KV / N bounds it')
        del r5
    clocks = sampler.summary(mark0, mark1) if sampler else None
    if sampler:
        sampler.stop()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = dict(metric=METRIC, value=res['value'], unit=UNIT, n_gpus=world, steps=K, warmup=max(args.warmup, 3),
                ms_per_step=res['ms_per_step'], higher_is_better=True, scaling='strong' if total else 'weak', vs_baseline=None,
                dtype='f16 weights and KV, f32 accumulate' + ('' if wl['batch'] // (world if total else 1) <= 16 else ' (activations rounded to f16 before the products above 16 sequences)'),
                data='synthetic',
                config=dict(workload=args.workload, **{k: v for k, v in wl.items() if k != 'total'}, batch_per_gpu=B, repeats=args.repeats,
                            steps_per_launch=min(args.per_launch, K), contexts=res['contexts'],
                            l2='weights + KV read per step (%.0f MB) exceed the 126 MB L2' % (res['roofline']['bytes_per_step'] / 1e6), cv=res['cv']),
                clocks=clocks, gpu_launches=res['gpu_launches'], e2e=res['e2e'], roofline=res['roofline'])
    if prefill:
        line['prefill'] = prefill
    if secondary:
        line['secondary'] = secondary
    if strong:
        line['strong'] = strong
    if extras and world == 1:
        torch.cuda.synchronize()
        line['ref_kernel'] = ref_kernel_block(args, ours_tokens)
    if not args.no_cpu_baseline and world == 1:
        P = wl['prompt']
        # a bounded sample: 16 consecutive steps of up to `cores` sequences through the reference interpreter (about 20 s);
        # the NumPy port for 10 s when no reference copy is installed
        ref = reference_interpreter() is not None
        r = cpu_steps_all_cores(sh, wl['batch'], P, 16 if ref else 2000, max_seconds=40 if ref else 10)
        line['cpu_baseline'] = dict(value=r['value'], unit=UNIT, cores=r['threads'], kind=r['kind'], sample=cpu_sample_text(r, wl, P))
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
