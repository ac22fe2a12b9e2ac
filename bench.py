"""Decode throughput of the Vesta GPT-2 step on B200, one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2] [--impl ours|reference]

A step is one decode step (one launch of the persistent kernel) of one batch. Protocol of the
reference benchmark (bench/g0_bench.py:166-180): reset, feed the prompt one token per step
(untimed), then time K generation steps that run back to back with the kernel feeding its own
token; the median of --repeats runs is reported. The prompt is a seeded uniform token sequence and
the weights are seeded random-init fp16 (the pretrained checkpoint and prompt need a download).

Workloads (BASELINE.json configs): cfg1 = GPT-2 small batch 1, cfg2 = batch 8 (the default: the
configuration the metric is quoted on), both 128-token prompts + 256 steps; cfg3 = batch 64 with
512-token prompts; xl1 / xl16 = XL shape at batch 1 / 16; cfg5 = 256 ragged sequences split over the
GPUs (strong scaling). With --gpus N > 1 every rank (one process per GPU, torchrun) runs its own
sequences (the same batch per GPU: weak scaling, except cfg5) with no exchange on the step path;
generated tokens are gathered to rank 0 at the end.

`value`   tokens/s with everything resident in HBM (CUDA events around the K launches)
`e2e`     tokens/s through the public API with host buffers: every step copies the input tokens
          from pinned host memory, launches, and reads the chosen tokens back
`roofline` algorithmic bytes per launch (all weights + attended K/V, the reference's byte model,
          vesta/gpt2.py:44-45,54-55) / mean launch duration, against the measured copy bandwidth
`cpu_baseline` the NumPy oracle (a port of the reference interpreter's arithmetic) on the host cores
"""
import argparse
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
# DRAM bytes (read + write) of one decode step from the ncu capture summarised in
# profiles/vesta_step_gpt2_small_b8.md, taken at the given context (attended positions per sequence). The bench's
# launches attend more positions: the K/V part is scaled by the positions, the weights are read once either way.
# Workloads that were not captured report null.
NCU_CAPTURE = {'cfg2': dict(bytes=291.1e6, positions=130)}


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

    def stop(self, start=0):
        if not self.proc:
            return None
        time.sleep(0.12)
        self.proc.terminate()
        rows = [r for r in self.rows[start:] if len(r) >= 7 and r[0].isdigit()] or \
               [r for r in self.rows if len(r) >= 7 and r[0].isdigit()]
        if not rows:
            return None
        sm = sorted(int(r[0]) for r in rows)
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        reasons = sorted({n for r in rows for n, v in zip(names, r[3:7]) if v.lower().startswith('active')})
        return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=int(rows[0][1]), reasons=reasons, samples=len(rows))


def host_threads():
    """let NumPy's BLAS use every host core (torchrun exports OMP_NUM_THREADS=1); -> the threads it then runs on"""
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=os.cpu_count())
        n = [int(i.get('num_threads', 1)) for i in threadpool_info()]
        return max(n) if n else 1
    except Exception:
        return 1


def cpu_baseline(sh, W, batch, ctx, steps, warm=1, max_seconds=None):
    """the NumPy oracle on the host: up to `steps` decode steps of one sequence starting at context ~ctx (the cache
    is filled with random fp16 values: the time does not depend on them), cut short after max_seconds.
    -> (steps per second, seconds, steps done)"""
    from oracle import gpt2_numpy as O
    rng = np.random.default_rng(0)
    room = min(ctx + steps + warm, sh.C)
    keys = (rng.standard_normal((sh.L, room, sh.H, sh.E), dtype=np.float32) * 0.1).astype(np.float16)
    vals = keys.copy()
    x = 1
    for t in range(warm):
        _, x = O.step(sh, W, keys, vals, x, min(ctx + t, room - 1))
    t0 = time.perf_counter()
    done = 0
    for t in range(steps):
        _, x = O.step(sh, W, keys, vals, x, min(ctx + warm + t, room - 1))
        done += 1
        if max_seconds and time.perf_counter() - t0 > max_seconds:
            break
    dt = time.perf_counter() - t0
    return done / dt, dt, done


def run_reference(args, wl, sh):
    """the reference arm: the CPU implementation of the path (NumPy port of vesta/interp.py's arithmetic
    for gpt2.vst) on the host cores, rank 0 only"""
    if int(os.environ.get('RANK', '0')) != 0:
        return
    from oracle import gpt2_numpy as O
    from vesta_gpu_b200.synth import make_weights
    W = O.upcast(make_weights(sh, 0))
    cores = host_threads()
    ctx = wl['prompt'] + wl['gen'] // 2
    # every step is one decode step of one sequence (a bounded sample of the batch); at most two minutes in all
    tps, dt, steps = cpu_baseline(sh, W, wl['batch'], ctx, max(1, args.steps), warm=max(1, min(args.warmup, 3)), max_seconds=120)
    sample = f'{steps} decode steps of one sequence at context {ctx} (of batch {wl["batch"]} x {wl["gen"]} steps), sequences run one after another'
    line = dict(metric=METRIC, value=tps, unit=UNIT, impl='reference', n_gpus=args.gpus, steps=steps, warmup=args.warmup,
                ms_per_step=1e3 * dt / steps / 1.0, higher_is_better=True, scaling='weak', vs_baseline=None,
                dtype='f32 accumulate over fp16-rounded weights', data='synthetic',
                config=dict(workload=args.workload, **wl),
                cpu_baseline=dict(value=tps, unit=UNIT, cores=cores, kind='port', sample=sample),
                e2e=dict(value=tps, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=256)
    ap.add_argument('--warmup', type=int, default=8)
    ap.add_argument('--repeats', type=int, default=5)
    ap.add_argument('--per-launch', type=int, default=16, help='decode steps inside one kernel launch (1: a launch per step)')
    ap.add_argument('--workload', default='cfg2', choices=sorted(WORKLOADS))
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--tune', default=None, help='JSON object of lowering options to override (experiments), e.g. {"kv_stages": 2}')
    args = ap.parse_args()
    from vesta_gpu_b200.shapes import SHAPES
    wl = dict(WORKLOADS[args.workload])
    sh = SHAPES[wl['shape']]
    if args.impl == 'reference':
        return run_reference(args, wl, sh)

    import torch
    import torch.distributed as dist
    from vesta_gpu_b200.synth import SynthGPT2, make_prompts
    from vesta_gpu_b200.gpt2 import VestaGPT2
    from vesta_gpu_b200.shard import gather_tokens

    rank, world = int(os.environ.get('RANK', '0')), int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    if world != args.gpus:
        raise SystemExit(f'--gpus {args.gpus} needs {args.gpus} ranks (torchrun --nproc-per-node {args.gpus}); WORLD_SIZE is {world}')
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    P, K, Wm = wl['prompt'], args.steps, max(args.warmup, 3)
    total = bool(wl.get('total'))
    if total and wl['batch'] % world:
        raise SystemExit(f'{wl["batch"]} sequences do not split over {world} GPUs')
    B = wl['batch'] // world if total else wl['batch']
    tmax = P + max(K, Wm) + 1
    if tmax > sh.C:
        raise SystemExit(f'prompt + steps = {tmax} exceeds the position table ({sh.C})')
    hf = SynthGPT2(sh, seed=0)
    tune = json.loads(args.tune) if args.tune else None
    ragged = wl.get('ragged')
    if ragged:
        from vesta_gpu_b200.synth import make_ragged_prompts
        from vesta_gpu_b200.shard import partition
        lens_all, toks_all = make_ragged_prompts(sh, B * world, ragged[0], ragged[1], seed=1)
        mine = partition(lens_all, world)[rank]
        lens, prompts = lens_all[mine], toks_all[mine]
        m = VestaGPT2(hf, batch=B, tmax=tmax, device=local, per_sequence_t=True, prompt_len=P, tune=tune)
        m.prompt.copy_(torch.from_numpy(prompts[:, :P].copy()))
        m.plen.copy_(torch.from_numpy(lens))
        start = torch.from_numpy((lens - P).astype(np.int32)).cuda()         # <= 0: every prompt ends at step P
        first_tok = torch.from_numpy(np.where(lens == P, prompts[:, 0], 0).astype(np.int32)).cuda()
        ctx_lens = [[int(n) + i + 1 for n in lens_all] for i in range(K)]    # attended positions of every sequence per step
    else:
        mine = list(range(rank * B, (rank + 1) * B))
        prompts = make_prompts(sh, B * world, P, seed=1)[rank * B:(rank + 1) * B]      # every rank its own sequences
        m = VestaGPT2(hf, batch=B, tmax=tmax, device=local, tune=tune)
        pd = torch.from_numpy(prompts.copy()).cuda()
        ctx_lens = [[P + i + 1] * (B * world) for i in range(K)]

    def prefill():
        m.reset()
        if ragged:
            # the kernel feeds itself from the prompt buffer; sequences start late so that all prompts end together
            m.t.copy_(start); m.x.copy_(first_tok)
            m.step(P)
        else:
            for t in range(P):
                m.x.copy_(pd[:, t])
                m.step()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # warm-up: prompt + Wm generation steps, untimed
    prefill(); m.step(Wm); torch.cuda.synchronize(); m.k.check()
    sampler = ClockSampler(local) if rank == 0 else None
    times, toks0 = [], None
    mark = 0
    for r in range(args.repeats):
        prefill()
        first = m.x.clone()
        sync_all()
        if r == 0 and sampler:
            mark = sampler.mark()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        m.k.launch(K, per_launch=args.per_launch)   # launches of per_launch steps back to back; the kernel feeds x and t itself
        e1.record()
        sync_all()
        times.append(e0.elapsed_time(e1) * 1e-3)
    m.k.check()
    # token streams of the last repeat, stepwise (untimed), for the gather and the e2e cross-check
    prefill()
    stream = [m.x.clone()]
    for _ in range(K - 1):
        m.step(); stream.append(m.x.clone())
    stream = torch.stack(stream, 1)
    torch.cuda.synchronize()

    # end to end: host buffers every step
    hx = torch.empty(B, dtype=torch.int32).pin_memory()
    hn = torch.empty(B, dtype=torch.float32).pin_memory()
    e2e_times = []
    for r in range(max(1, min(3, args.repeats))):
        prefill()
        hx.copy_(m.x.cpu())
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        seen = []
        for _ in range(K):
            # host -> device: this step's input tokens; one launch; device -> host: the chosen tokens; synchronise
            m.step_host(hx, hn)
            hx.copy_(hn.to(torch.int32))
            seen.append(hx.clone())
        e1.record()
        sync_all()
        e2e_times.append(e0.elapsed_time(e1) * 1e-3)
    # after K host-driven steps hx holds the token chosen by generation step K; the device loop's stream
    # holds the tokens before steps 1..K, so its last column is the token chosen by step K-1
    e2e_ok = None
    if K > 1:
        # fraction of the host-driven stream equal to the device-fed one (fp32 atomics make the last bits, and
        # hence near-ties over hundreds of free-running steps, run-dependent)
        e2e_ok = round(float((torch.stack(seen[:-1], 1) == stream[:, 1:].cpu()).float().mean()), 4)
    clocks = sampler.stop(mark) if sampler else None

    med = statistics.median(times)
    e2e_med = statistics.median(e2e_times)
    if world > 1:
        tt = torch.tensor([med, e2e_med], device='cuda', dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        med, e2e_med = float(tt[0]), float(tt[1])
    all_tokens = gather_tokens(stream.to(torch.int32), list(mine), B * world)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    assert all_tokens.shape == (B * world, K)

    # algorithmic bytes of one launch on one GPU: every weight once + the attended K/V of its sequences
    bytes_per_step = sum(sh.weight_bytes() + sh.kv_bytes_per_pos() * sum(c) / world for c in ctx_lens) / K
    peak, peak_src = peaks()
    achieved = bytes_per_step / (med / K) / 1e9
    spl = min(args.per_launch, K)
    cap = NCU_CAPTURE.get(args.workload) if world == 1 else None
    traffic = None
    if cap:
        mean_pos = sum(sum(c) for c in ctx_lens) / K / (B * world)
        traffic = (cap['bytes'] + B * (mean_pos - cap['positions']) * sh.kv_bytes_per_pos()) * spl
    line = dict(metric=METRIC, value=B * world * K / med, unit=UNIT, n_gpus=world, steps=K, warmup=Wm,
                ms_per_step=1e3 * med / K, higher_is_better=True, scaling='strong' if total else 'weak', vs_baseline=None,
                dtype='f16 weights and KV, f32 accumulate', data='synthetic',
                config=dict(workload=args.workload, **{k: v for k, v in wl.items() if k != 'total'}, batch_per_gpu=B, repeats=args.repeats, steps_per_launch=min(args.per_launch, K), **({'tune': tune} if tune else {}),
                            l2='weights + KV read per step (%.0f MB) exceed the 126 MB L2' % (bytes_per_step / 1e6),
                            cv=round(statistics.pstdev(times) / statistics.mean(times), 4)),
                clocks=clocks, gpu_launches=-(-K // args.per_launch),
                e2e=dict(value=B * world * K / e2e_med, unit=UNIT, h2d_bytes_per_step=B * 4, d2h_bytes_per_step=B * 4,
                         tokens_match_device_loop=e2e_ok),
                roofline=dict(bound='hbm', achieved=achieved, peak=peak, unit='GB/s', frac=achieved / peak, traffic=traffic,
                              peak_source=peak_src, bytes_per_step=bytes_per_step, bytes_per_launch=bytes_per_step * spl, kernel='vesta_step',
                              frac_of_8tbs=achieved / 8000.0))
    if not args.no_cpu_baseline and world == 1:
        from oracle import gpt2_numpy as O
        cores = host_threads()
        ctx = P + K // 2
        # a bounded sample: about 12 seconds of decode steps of one sequence
        tps, dt, nsteps = cpu_baseline(sh, O.upcast(hf.weights), B, ctx, 2000, max_seconds=12)
        line['cpu_baseline'] = dict(value=tps, unit=UNIT, cores=cores, kind='port',
                                    sample=f'{nsteps} decode steps of one sequence at context {ctx}, NumPy oracle, {dt:.1f} s')
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
