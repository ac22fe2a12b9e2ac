"""Placement of a decode-step program on the 148 SMs of a B200 and assembly of the CUDA source
of ONE persistent cooperative kernel (plus a one-time weight-packing kernel).

    lower(text, res, axis_max, batch=1, per_token=(), outputs=(), feedback=None, timing=False) -> Lowered

Same call and the same Lowered fields as the reference compiler (vesta/lower.py:1294-1329,
69-79), so vesta.gpt2-style callers and Kernel.view() work unchanged. What happens inside is
different by design: instead of deriving scalar CUDA C statement by statement, this pass

  1. recognises the program: every statement is matched, in order, against the statement
     patterns of the decode-step family (embed; per layer LN -> QKV -> KV emit -> scores ->
     softmax -> PV -> projection + residual -> LN -> FC -> tanh-GELU -> projection + residual;
     then LN -> tied-embedding logits -> argmax with lowest-id ties). Names, sizes and
     constants are read from the program; anything that does not match raises
     NotImplementedError (there is no generic or CPU fallback by design);
  2. places the five contractions on the CTAs of a one-CTA-per-SM grid (NARROW: whole fold, a few
     output tiles per CTA; WIDE: a slice of the fold for many output tiles, combined by atomics),
     balancing the bytes every CTA streams per step, and lays each CTA's share of the fp16 weights
     out as one contiguous stream of mma-ordered 16x16 tiles (Lowered.place, consumed by the
     packing kernel and the step kernel);
  3. prepends the sizes, placement constants and the kernel signatures to the hand-written
     sm_100a kernel text in csrc/step_kernel.cuh.
"""
import math
from dataclasses import dataclass, field, fields, is_dataclass
from pathlib import Path

import numpy as np

from . import syntax as sx

CSRC = Path(__file__).resolve().parent / 'csrc'
COMMON_TEXT = CSRC / 'step_common.cuh'
KERNEL_TEXT = CSRC / 'step_kernel.cuh'          # batches above eight sequences
SMALL_TEXT = CSRC / 'step_small.cuh'            # at most eight sequences: one batch tile

CTYPE = {'f32': 'float', 'f16': 'unsigned short', 'i32': 'int'}
NW = 8                 # consumer warps per CTA (one more warp streams the weights)
WG = 2 * NW            # output tiles per unit of the attention projection (placement)
CHUNK_TILES = 32       # ring slots of at least 16 KB (a slot holds at least one row of a WIDE group)
WN_MAX = 4             # widest NARROW placement
PT_STRIDE = 16
SMEM_LIMIT = 227 * 1024
DEFAULT_SMS = 148      # B200


@dataclass
class Lowered:
    src: str
    params: list             # (name, dtype, emitted) in kernel argument order
    scratch: dict            # host-visible name -> (offset, axes, static shape)
    scratch_floats: int
    shared_bytes: int        # dynamic shared memory per block
    barriers_per_launch: int
    plan: list = field(default_factory=list)     # (statement, placement) for reading
    sites: list = field(default_factory=list)    # timing: what each TS slot measures
    counters: int = 2                            # length of the bar array
    # additions of this backend
    block: int = (NW + 1) * 32                   # threads per CTA
    grid: int = DEFAULT_SMS                      # CTAs the placement was made for (one per SM)
    place: np.ndarray = None                     # int32 [grid, PT_STRIDE] placement records
    packed_bytes: int = 0                        # size of the packed weight copy
    pack_params: list = field(default_factory=list)   # residues the packing kernel reads
    dims: dict = field(default_factory=dict)     # sizes and constants read from the program
    roles: dict = field(default_factory=dict)    # role -> residue name


# ------------------------------------------------------------------ recognition
class Mismatch(Exception):
    pass


def _unify(pat, node, env):
    """structural match of a pattern tree against a program tree; `$name` binds"""
    if isinstance(pat, str):
        if pat.startswith('$'):
            if pat in env and env[pat] != node:
                raise Mismatch(f'{pat} is {env[pat]!r}, found {node!r}')
            env[pat] = node
            return
        if pat != node:
            raise Mismatch(f'expected {pat!r}, found {node!r}')
        return
    if isinstance(pat, sx.Name) and pat.id.startswith('$'):
        if isinstance(node, sx.Name):
            return _unify(pat.id, node.id, env)
        if isinstance(node, sx.Num):
            return _unify(pat.id, node.value, env)
        raise Mismatch(f'{pat.id} cannot stand for {type(node).__name__}')
    if isinstance(pat, tuple):
        if not isinstance(node, tuple) or len(pat) != len(node):
            raise Mismatch('different number of indices or statements')
        for p, n in zip(pat, node):
            _unify(p, n, env)
        return
    if is_dataclass(pat):
        if type(pat) is not type(node):
            raise Mismatch(f'expected {type(pat).__name__}, found {type(node).__name__}')
        for f in fields(pat):
            _unify(getattr(pat, f.name), getattr(node, f.name), env)
        return
    if pat != node:
        raise Mismatch(f'expected {pat!r}, found {node!r}')


def _pattern(text):
    stmts = sx.parse(text, wild=True)
    assert len(stmts) == 1, text
    return stmts[0]


# statements of the layer body, in order; Q numbers refer to the questions of the reference
# (QUESTIONS.md:15-88, vesta/programs/gpt2.vst:37-72)
LAYER_PATTERNS = [
    ('LN1 mean', '$m1 = fold sum $d: $z[$d] / $D'),
    ('LN1 variance', '$v1 = fold sum $d: ($z[$d] - $m1) * ($z[$d] - $m1) / $D'),
    ('LN1', '$a[$d] = ($z[$d] - $m1) / sqrt($v1 + $eps) * $ln1w[$l, $d] + $ln1b[$l, $d]'),
    ('QKV', '$qkv[$j] = (fold sum $d: $a[$d] * $qkvw[$l, $d, $j]) + $qkvb[$l, $j]'),
    ('query view', '$q[$h, $e] = $qkv[$h * $E + $e]'),
    ('K emit', 'residue $keys[$l, $t, $h, $e] <- $qkv[$D + $h * $E + $e]'),
    ('V emit', 'residue $vals[$l, $t, $h, $e] <- $qkv[$D2 + $h * $E + $e]'),
    ('scores', '$sc[$h, $s] = (fold sum $e: $q[$h, $e] * $keys[$l, $s, $h, $e]) / $scale'),
    ('softmax max', '$mx[$h] = fold max $s: $sc[$h, $s]'),
    ('softmax exp', '$ex[$h, $s] = exp($sc[$h, $s] - $mx[$h])'),
    ('softmax weights', '$w[$h, $s] = $ex[$h, $s] / (fold sum $s: $ex[$h, $s])'),
    ('PV', '$o[$h, $e] = fold sum $s: $w[$h, $s] * $vals[$l, $s, $h, $e]'),
    ('attn-proj', '$oo[$d] = fold sum $h: (fold sum $e: $o[$h, $e] * $ow[$l, $h * $E + $e, $d])'),
    ('residual 1', '$z1[$d] = $z[$d] + $oo[$d] + $ob[$l, $d]'),
    ('LN2 mean', '$m2 = fold sum $d: $z1[$d] / $D'),
    ('LN2 variance', '$v2 = fold sum $d: ($z1[$d] - $m2) * ($z1[$d] - $m2) / $D'),
    ('LN2', '$b[$d] = ($z1[$d] - $m2) / sqrt($v2 + $eps) * $ln2w[$l, $d] + $ln2b[$l, $d]'),
    ('FC', '$u[$f] = (fold sum $d: $b[$d] * $fcw[$l, $d, $f]) + $fcb[$l, $f]'),
    ('GELU', '$g[$f] = $ga * $u[$f] * ($one + tanh($gb * ($u[$f] + $gc * $u[$f] * $u[$f] * $u[$f])))'),
    ('MLP-proj + residual 2', '$z2[$d] = $z1[$d] + (fold sum $f: $g[$f] * $pw[$l, $f, $d]) + $pb[$l, $d]'),
]
# The additive parameters (the shifts of the three LayerNorms, the biases of the four contractions) may be absent from a
# program: the statement is then matched without its last term and the kernel reads a vector of zeros in its place.
OPTIONAL_TERMS = {
    'LN1': (' + $ln1b[$l, $d]', 'ln1b'), 'QKV': (' + $qkvb[$l, $j]', 'qkvb'), 'residual 1': (' + $ob[$l, $d]', 'ob'),
    'LN2': (' + $ln2b[$l, $d]', 'ln2b'), 'FC': (' + $fcb[$l, $f]', 'fcb'), 'MLP-proj + residual 2': (' + $pb[$l, $d]', 'pb'),
    'LNf': (' + $lnfb[$d]', 'lnfb'),
}
ZEROS = '_zeros'                 # name of the kernel parameter that stands in for absent additive parameters
HEAD_PATTERNS = [
    ('LNf mean', '$m3 = fold sum $d: $zL[$d] / $D'),
    ('LNf variance', '$v3 = fold sum $d: ($zL[$d] - $m3) * ($zL[$d] - $m3) / $D'),
    ('LNf', '$c[$d] = ($zL[$d] - $m3) / sqrt($v3 + $eps) * $lnfw[$d] + $lnfb[$d]'),
    ('logits', '$logit[$n] = fold sum $d: $c[$d] * $wte[$n, $d]'),
    ('best', '$best = fold max $n: $logit[$n]'),
    ('next', '$next = fold min $n: fork $logit[$n] == $best ? $n : $N'),
]
EMBED_PATTERN = ('embed', '$z0[$d] = $wte[$x, $d] + $wpe[$t, $d]')


def _show(node):
    return getattr(node, 'name', type(node).__name__)


def recognise(text):
    """program text -> (env of bindings, axis extents, received residues {name: axes})"""
    stmts = sx.parse(text)
    axes, recv, rest = {}, {}, []
    for s in stmts:
        if isinstance(s, sx.AxisDef):
            axes[s.name] = s.extent
        elif isinstance(s, sx.Receive):
            recv[s.name] = s.axes
        else:
            rest.append(s)
    env = {}

    def need(label, pat_text, node):
        trial = dict(env)
        try:
            _unify(_pattern(pat_text), node, trial)
        except Mismatch as err:
            term, role = OPTIONAL_TERMS.get(label, (None, None))
            if term and pat_text.endswith(term):
                trial = dict(env)
                try:
                    _unify(_pattern(pat_text[:-len(term)]), node, trial)
                except Mismatch:
                    trial = None
                if trial is not None:
                    trial['$' + role] = None              # absent: zeros
                    env.clear(); env.update(trial)
                    return
            raise NotImplementedError(
                f'statement {_show(node)!r} is not the {label} statement of a decode step: {err}') from None
        env.clear(); env.update(trial)

    if len(rest) != 2 + len(HEAD_PATTERNS) or not isinstance(rest[1], sx.StepFold):
        raise NotImplementedError('not a decode-step program: expected embed, one `fold step` over the layers, '
                                  f'then {len(HEAD_PATTERNS)} head statements')
    need(*EMBED_PATTERN, rest[0])
    step = rest[1]
    try:
        _unify(sx.StepFold('$zL', ('$d',), '$l', sx.Name('$z0'), '$z', step.body, sx.Name('$z2')), step, env)
    except Mismatch as err:
        raise NotImplementedError(f'layer loop: {err}') from None
    if len(step.body) != len(LAYER_PATTERNS):
        raise NotImplementedError(f'layer body has {len(step.body)} statements, a decode step has {len(LAYER_PATTERNS)}')
    for (label, pat), node in zip(LAYER_PATTERNS, step.body):
        need(label, pat, node)
    for (label, pat), node in zip(HEAD_PATTERNS, rest[2:]):
        need(label, pat, node)

    ext = {}
    for name, e in axes.items():
        if isinstance(e, sx.Num):
            ext[name] = int(e.value)
        elif e == sx.Bin('+', sx.Name(env['$t']), sx.Num(1)):
            ext[name] = None                      # run-time extent: positions seen so far
        else:
            raise NotImplementedError(f'axis {name}: extent must be a number or {env["$t"]} + 1')
    return env, ext, recv


def _dims(env, ext):
    g = lambda k: ext[env[k]]
    D, H, E, F, N, J, L = g('$d'), g('$h'), g('$e'), g('$f'), g('$n'), g('$j'), g('$l')
    checks = [
        (ext[env['$s']] is None, 'the position axis must have the run-time extent t + 1'),
        (env['$D'] == D, 'LayerNorm divides by the width'),
        (H * E == D, 'heads x head width must equal the width'),
        (env['$E'] == E, 'head views must use the head width'),
        (J == 3 * D and env['$D2'] == 2 * D, 'QKV must be three width-sized parts'),
        (env['$N'] == N, 'the argmax default must be the vocabulary size'),
        (env['$one'] == 1, 'GELU form'),
        (D % 16 == 0 and F % 16 == 0 and E % 8 == 0, 'width and MLP width must be multiples of 16, head width of 8'),
        (E == 64, 'this kernel holds one 128-byte K/V row per 8 lanes: head width 64'),
    ]
    for ok, why in checks:
        if not ok:
            raise NotImplementedError(f'program outside the supported family: {why}')
    return dict(D=D, H=H, E=E, F=F, N=N, J=J, L=L, eps=float(env['$eps']), scale=float(env['$scale']),
                gelu=(float(env['$ga']), float(env['$gb']), float(env['$gc'])))


ROLE_KEYS = ('x', 't', 'wte', 'wpe', 'ln1w', 'ln1b', 'qkvw', 'qkvb', 'ow', 'ob', 'ln2w', 'ln2b',
             'fcw', 'fcb', 'pw', 'pb', 'lnfw', 'lnfb', 'keys', 'vals')


# ------------------------------------------------------------------ placement
def _spread(total, loads, cap):
    """hand out `total` equal units one at a time to the least loaded CTA (at most cap each);
    -> counts per CTA. loads is updated by the caller's unit weight afterwards."""
    counts = [0] * len(loads)
    cur = list(loads)
    for _ in range(total):
        c = min((i for i in range(len(cur)) if counts[i] < cap), key=lambda i: (cur[i], i), default=None)
        if c is None:
            raise NotImplementedError('placement: too many output tiles for this grid')
        counts[c] += 1
        cur[c] += 1.0
    return counts


def place_step(dims, grid, ksplit=False):
    """-> (int32 [grid, PT_STRIDE] placement records, tiles per CTA stream, plan notes). ksplit: the MLP projection
    as units of two output tiles x a slice of the fold (as few slices as fill the grid), independent of where the
    FC tiles are"""
    D, F, N, L = dims['D'], dims['F'], dims['N'], dims['L']
    KT_D, KT_F, JT_D, JT_J, JT_N = D // 16, F // 16, D // 16, 3 * D // 16, (N + 15) // 16
    G = grid
    # FC / MLP-proj: every f tile costs 2*KT_D tiles of stream; at most WN_MAX per CTA
    fc = _spread(KT_F, [0.0] * G, WN_MAX)
    load = [(1.0 if ksplit else 2.0) * KT_D * n for n in fc]
    # QKV: every output tile costs KT_D tiles of stream. The phases are separated by grid barriers, so what a phase
    # costs is its largest share: no CTA gets more than ceil(tiles / CTAs) of them; within that, the CTAs with the
    # fewest bytes so far come first.
    cap = min(WN_MAX, max(1, math.ceil(JT_J / G)))
    if JT_J > cap * G:
        raise NotImplementedError('placement: too many QKV output tiles for this grid')
    cnt = [0] * G
    for _ in range(JT_J):
        c = min((i for i in range(G) if cnt[i] < cap), key=lambda i: (load[i], i))
        cnt[c] += 1
        load[c] += KT_D
    qkv = cnt

    def units_of(kt, wj):
        """output tiles in groups of wj x slices of a fold of kt tiles, one unit per CTA"""
        groups = math.ceil(JT_D / wj)
        splits = max(1, min(kt, G // groups))
        nk = math.ceil(kt / splits)
        us = [(jg * wj, min(wj, JT_D - jg * wj), k0, min(nk, kt - k0)) for jg in range(groups) for k0 in range(0, kt, nk)]
        if len(us) > G:
            raise NotImplementedError('placement: projection units exceed the grid')
        return us, nk

    def deal(us):
        out = [None] * G
        order = sorted(range(G), key=lambda i: (load[i], i))
        for u, c in zip(us, order):
            out[c] = u
            load[c] += u[1] * u[3]
        return out
    # attn-proj: groups of WG output tiles x slices of the fold, one unit per CTA
    units, nk = units_of(KT_D, WG)
    proj = deal(units)
    p2 = [None] * G
    p2_nk = 0
    if ksplit:
        units2, p2_nk = units_of(KT_F, 2)
        p2 = deal(units2)
    # logits: output tiles over the whole fold, the same number per CTA (the phase costs its largest share); the
    # CTAs with the fewest bytes in the layers take the remainder
    step_load = [L * v for v in load]
    cnt = [JT_N // G] * G
    for c in sorted(range(G), key=lambda i: (step_load[i], i))[:JT_N % G]:
        cnt[c] += 1
    logit = cnt

    rec = np.zeros((G, PT_STRIDE), np.int32)
    base = 0
    fj = qj = lj = 0
    for c in range(G):
        pj0, pnj, pk0, pnk = proj[c] or (0, 0, 0, 0)
        qj0, qnj, qk0, qnk = p2[c] or (0, 0, 0, 0)
        layer = qkv[c] * KT_D + pnj * pnk + fc[c] * KT_D + (qnj * qnk if ksplit else JT_D * fc[c])
        rec[c, :12] = (base, layer, qj, qkv[c], pj0, pnj, pk0, pnk, fj, fc[c], lj, logit[c])
        rec[c, 12:16] = (qj0, qnj, qk0, qnk)
        qj += qkv[c]; fj += fc[c]; lj += logit[c]
        base += L * layer + logit[c] * KT_D
    assert qj == JT_J and fj == KT_F and lj == JT_N
    if base >= 2 ** 31:
        raise NotImplementedError('packed weights exceed the 32-bit tile index')
    per = rec[:, 1].astype(np.int64) * L + rec[:, 11].astype(np.int64) * KT_D
    notes = dict(tiles_total=int(base), tiles_min=int(per.min()), tiles_max=int(per.max()),
                 tiles_mean=float(per.mean()), proj_units=len(units), proj_nk=nk, p2_nk=p2_nk)
    return rec, int(base), notes


# ------------------------------------------------------------------ assembly

def _entry_points(res, roles, fb, prompt_len, row_seq=False):
    """-> (params, pack_params, text of the two extern "C" kernels that wrap step_body / pack_body)"""
    emitted = {roles['keys'], roles['vals']} | (set(fb) if fb else set())
    params, sig = [], []
    for name, (shape, dt) in res.items():
        em = name in emitted
        params.append((name, dt, em))
        sig.append(f'{"" if em else "const "}{CTYPE[dt]}* __restrict__ R_{name}')
    if prompt_len and fb:
        params += [('prompt', 'i32', False), ('plen', 'i32', False)]
        sig += ['const int* __restrict__ X_prompt', 'const int* __restrict__ X_plen']
    if row_seq:
        params += [('row_seq', 'i32', False)]
        sig += ['const int* __restrict__ X_row_seq']
    if ZEROS in roles.values():
        # additive parameters the program does not have: one vector of zeros (allocated by Kernel.bind) stands for all
        params += [(ZEROS, 'f16', False)]
        sig += ['const unsigned short* __restrict__ X_zeros']
    R = {k: ('X_zeros' if v == ZEROS else 'R_' + v) for k, v in roles.items()}
    step_sig = ', '.join(sig + ['float* __restrict__ S', 'unsigned* bar', 'unsigned long long* TS',
                                'const unsigned char* __restrict__ WP', 'const int* __restrict__ PT',
                                'const unsigned char* __restrict__ TM', 'int nsteps'])
    fill = [f'a.x = {R["x"]}; a.t = {R["t"]};']
    for k in ('wte', 'wpe', 'ln1w', 'ln1b', 'qkvb', 'ob', 'ln2w', 'ln2b', 'fcb', 'pb', 'lnfw', 'lnfb'):
        fill.append(f'a.{k} = {R[k]};')
    fill.append(f'a.keys = {R["keys"]}; a.vals = {R["vals"]};')
    if fb:
        fill.append(f'a.x_out = {R["x"]}; a.t_out = {R["t"]};')
    else:
        fill.append('a.x_out = 0; a.t_out = 0;')
    fill.append('a.prompt = X_prompt; a.plen = X_plen;' if (prompt_len and fb) else 'a.prompt = 0; a.plen = 0;')
    fill.append('a.row_seq = X_row_seq;' if row_seq else 'a.row_seq = 0;')
    fill.append('a.S = S; a.bar = bar; a.TS = TS; a.WP = WP; a.PT = PT; a.TM = TM; a.nsteps = nsteps;')
    pack_roles = ('wte', 'qkvw', 'ow', 'fcw', 'pw')
    pack_params = [roles[k] for k in pack_roles]
    pack_sig = ', '.join([f'const unsigned short* __restrict__ R_{roles[k]}' for k in pack_roles]
                         + ['unsigned char* __restrict__ WP', 'const int* __restrict__ PT'])
    pack_fill = ' '.join(f'p.{k} = R_{roles[k]};' for k in pack_roles) + ' p.WP = WP; p.PT = PT;'
    tail = (f'\nextern "C" __global__ void __launch_bounds__(NTHREADS, 1) vesta_step({step_sig}) {{\n'
            f'    Args a; {" ".join(fill)}\n    step_body(a);\n}}\n'
            f'\nextern "C" __global__ void vesta_pack({pack_sig}) {{\n'
            f'    PackArgs p; {pack_fill}\n    pack_body(p);\n}}\n')
    return params, pack_params, tail


def _f32(v):
    return repr(float(np.float32(v))) + 'f'


def _up(v, a=64):
    return (v + a - 1) // a * a


def _lower_small(env, dims, res, roles, fb, B, tmax, cpos, t_per_token, t_name, prompt_len, timing, grid, tune):
    """at most eight sequences: the kernel text csrc/step_small.cuh (one batch tile, fold split over the warps of a CTA
    for QKV and FC, whole output tiles per warp for the projections, attention tiles listed once per step)"""
    D, H, E, F, N, L = dims['D'], dims['H'], dims['E'], dims['F'], dims['N'], dims['L']
    KT_D = D // 16
    nw = int(tune.get('warps', NW))                 # consumer warps per CTA
    rec, tiles, notes = place_step(dims, grid, False)
    wn = max(int(rec[:, 3].max()), int(rec[:, 9].max()), 1)              # most output tiles of a whole-fold contraction per CTA
    umax = max(int(rec[:, 7].max()), int(rec[:, 9].max()), 1)            # deepest fold slice of a projection unit
    if umax > 8:
        raise NotImplementedError('placement: a projection unit is deeper than eight fold tiles')

    # position chunks per (sequence, head), from the measured costs of the attention phase (cycles): an item costs a fixed
    # 1,500 plus 1,300 per tile of 128 positions, a CTA runs its items one after the other, and the projection that
    # follows merges the chunks of a pair at about 80 per chunk; sized for a full cache
    def att_cost(k):
        return math.ceil(B * H * k / grid) * (1500 + 1300 * math.ceil(math.ceil(tmax / k) / 128)) + 80 * k
    nch = int(tune.get('nch', min(range(1, 17), key=lambda k: (att_cost(k), k))))
    # One chunk per (sequence, head): the CTA that finishes an item also applies the head's 64 rows of the attention
    # projection (streamed behind the item's K/V tiles) and adds the result into z1; the projection phase and its grid
    # barrier disappear. With several chunks per pair the partial results have to be merged first, by a phase of its own.
    fuse = bool(tune.get('fuse_proj', nch == 1))
    if fuse:
        nch = 1
        fus = E // 16                                                    # fold tiles of one head
        # the per-CTA streams lose their projection segment; the heads' slices follow them, one copy each (items of the
        # same head on different CTAs read the same tiles: from L2 after the first)
        base = 0
        for c in range(grid):
            rec[c, 4:8] = 0
            layer = int(rec[c, 3]) * KT_D + int(rec[c, 9]) * KT_D + (D // 16) * int(rec[c, 9])
            rec[c, 0], rec[c, 1] = base, layer
            base += L * layer + int(rec[c, 11]) * KT_D
        fuse_base = base
        base += L * H * (D // 16) * fus
        if base >= 2 ** 31:
            raise NotImplementedError('packed weights exceed the 32-bit tile index')
        tiles = base
        umax = max(int(rec[:, 9].max()), fus)
        notes = dict(notes, proj_units=B * H, proj_nk=fus, tiles_total=int(base))
    att_items = B * H * nch
    # Fused projection with an exchange inside the head: where every CTA has at most one item, the B CTAs that hold the
    # items of one head pass their 64 outputs through global memory (tagged values, nobody else waits) and each
    # applies 1 / B of the head's output tiles to all B sequences: the head's rows of the projection are then read once
    # per head, not once per item (at eight sequences 12 KB per CTA instead of 96 KB through the ring).
    fuse_x = bool(fuse and tune.get('fuse_exchange', True) and 2 <= B and B * H <= grid)
    # ... and the same way from the QKV phase to the attention items: query, K and V of the current position travel as
    # tagged values, the grid barrier between the two phases goes (two barriers per layer)
    # (also without the fused projection, at one or two sequences, where the pairs are cut into chunks: one item per CTA
    # is all it takes)
    fuse_x2 = bool(tune.get('qkv_exchange', True) and att_items <= grid and (fuse_x or not fuse))
    # ... and, without the fused projection, from the attention items to the projection phase (their partial results)
    fuse_x3 = bool(fuse_x2 and not fuse and tune.get('part_exchange', True))
    maxtl = math.ceil(att_items / grid) * math.ceil(math.ceil(tmax / nch) / 128)
    # K/V stages of 32 KB: two tiles in flight where a CTA has several per layer, one (and a deeper weight ring) otherwise
    kvst = int(tune.get('kv_stages', 2 if maxtl > 1 else 1))

    off_logit, off_next = 0, _up(B * N)
    # state vectors as 64-bit fixed point combined with integer atomics: bit-identical runs. Free at one or two sequences
    # (measured: 194 us per step either way at batch 1), 11 % slower at eight (260 against 234 us), so opt-in there
    fixed_sums = bool(tune.get('ordered', B <= 2))
    off_z = _up(off_next + B)
    off_q = off_z + 3 * _up(B * D) * (2 if fixed_sums else 1)
    off_part = off_q + _up(B * D)
    off_x = off_part + _up(att_items * (E + 2) * (2 if fuse_x3 else 1))    # (fuse_x3: the partial results as (value, tag) pairs); exchange buffers of such pairs:
    off_best = off_x + _up(2 * H * B * E * (int(fuse_x) + 3 * int(fuse_x2)))   # the heads' outputs (fuse_x), then query, K and V rows (fuse_x2)
    scratch_floats = off_best + _up(2 * B)
    scratch = {env['$logit']: (off_logit, ('bt', env['$n']), (B, N)), env['$next']: (off_next, ('bt',), (B,))}

    # shared memory: [weight ring | K/V stages | operand tiles | GELU operand tiles | partial sums | parameters | misc | barriers]
    ch = CHUNK_TILES
    budget = SMEM_LIMIT - (9216 if timing else 0)
    prm_bytes = 10 * D + wn * 32               # gain and shift as fp32, two bias vectors as fp16
    misc_bytes = 2 * nw * (E + 2) * 4 + 8 * nw * 8 + 32 + 512 + 16 + maxtl * 16
    fixed = kvst * 32768 + KT_D * 576 + _up(max(wn, E // 16 if fuse else 0) * 576, 128) + nw * wn * 512 + _up(prm_bytes, 16) + _up(misc_bytes, 16)
    nslot = min((budget - fixed - 2 * kvst * 8 - 64) // (ch * 512 + 16), 16)
    if nslot < 2:
        raise NotImplementedError('model too wide for the shared-memory budget')
    sm_ring = 0
    sm_kv = sm_ring + nslot * ch * 512
    sm_act = sm_kv + kvst * 32768
    sm_gact = sm_act + KT_D * 576
    sm_red = sm_gact + _up(max(wn, E // 16 if fuse else 0) * 576, 128)
    sm_prm = sm_red + nw * wn * 512
    sm_misc = sm_prm + _up(prm_bytes, 16)
    sm_bars = sm_misc + _up(misc_bytes, 16)
    shared = sm_bars + (2 * nslot + 2 * kvst) * 8

    scale = dims['scale']
    defs = dict(V_NW=nw, V_NPROD=2, V_B=B, V_L=L, V_D=D, V_H=H, V_E=E, V_F=F, V_N=N, V_TMAX=tmax, V_CPOS=cpos,
                V_EPS=_f32(dims['eps']), V_SCALE=_f32(scale), V_SCALE_IS_POW2=int(math.frexp(scale)[0] == 0.5),
                V_GELU_A=_f32(dims['gelu'][0]), V_GELU_B=_f32(dims['gelu'][1]), V_GELU_C=_f32(dims['gelu'][2]),
                V_NSLOT=nslot, V_CH=ch, V_KVST=kvst, V_UMAX=umax, V_WN=wn, V_FIXED=int(fixed_sums), V_FUSE_PROJ=int(fuse), V_FUSE_X=int(fuse_x), V_FUSE_X2=int(fuse_x2), V_FUSE_X3=int(fuse_x3), V_FUSE_BASE=(fuse_base if fuse else 0), V_NCH=nch, V_MAXTL=maxtl, V_MAXGRID=grid,
                V_TSTRIDE=int(t_per_token), V_FEEDBACK=int(bool(fb)), V_TSTEP=int(fb.get(t_name, 0)),
                V_TIMING=int(timing), V_PLEN=int(prompt_len) if fb else 0,
                V_OFF_LOGIT=off_logit, V_OFF_NEXT=off_next, V_OFF_Z=off_z, V_OFF_Q=off_q, V_OFF_PART=off_part, V_OFF_X=off_x, V_OFF_BEST=off_best,
                V_SM_RING=sm_ring, V_SM_KV=sm_kv, V_SM_ACT=sm_act, V_SM_GACT=sm_gact, V_SM_RED=sm_red, V_SM_PRM=sm_prm,
                V_SM_MISC=sm_misc, V_SM_BARS=sm_bars,
                V_WAIT_NS=f"{int(tune.get('wait_ns', 500_000_000))}ull")
    head = ''.join(f'#define {k} {v}\n' for k, v in defs.items())
    params, pack_params, tail = _entry_points(res, roles, fb, prompt_len)
    src = head + COMMON_TEXT.read_text(encoding='utf-8') + SMALL_TEXT.read_text(encoding='utf-8') + tail

    q = env
    ln_how = (f'every CTA recomputes: {nw // (1 if B <= 1 else 2 if B <= 2 else 4 if B <= 4 else 8)} warp(s) per row, the row in registers, '
              'into mma operand tiles (fp16 head + fp16 remainder)')
    plan = [
        (f'{q["$z0"]} (embed)', 'grid-stride, then barrier'),
        (f'{q["$m1"]}, {q["$v1"]}, {q["$a"]} (LN1)', ln_how),
        (f'{q["$qkv"]} + emits', f'whole fold, {min(rec[:, 3])}-{max(rec[:, 3])} output tiles per CTA, the fold split over the {nw} warps; bias, q, K/V emit in the epilogue'),
        (f'{q["$sc"]}, {q["$mx"]}, {q["$ex"]}, {q["$w"]}, {q["$o"]} (attention)',
         f'one item per (sequence, head, 1/{nch} of the positions), dealt round-robin over the CTAs, cut into tiles of 128 positions once per step; '
         f'K/V tiles by TMA ({kvst} stages), online softmax in registers, merged by the projection'),
        (f'{q["$oo"]}, {q["$z1"]}', (f'per (sequence, head) item, by the CTA that finished its attention: the head\'s {E} rows of the projection x all output tiles, fp32 atomics into {q["$z1"]} (no phase of its own)' if fuse
                                      else f'fold slices: {notes["proj_units"]} units of up to {WG} output tiles x {notes["proj_nk"]} fold tiles, whole output tiles per warp, fp32 atomics')),
        (f'{q["$m2"]}, {q["$v2"]}, {q["$b"]} (LN2)', ln_how),
        (f'{q["$u"]}, {q["$g"]}', f'whole fold, {min(rec[:, 9])}-{max(rec[:, 9])} f tiles per CTA, GELU in the epilogue, result stays in shared memory'),
        (f'{q["$z2"]}', 'fold slice = the CTA\'s own f tiles, whole output tiles per warp, fp32 atomics'),
        (f'{q["$m3"]}, {q["$v3"]}, {q["$c"]} (LNf)', ln_how),
        (f'{q["$logit"]}', f'whole fold, {min(rec[:, 11])}-{max(rec[:, 11])} vocabulary tiles per CTA in groups of 16, two per warp'),
        (f'{q["$best"]}, {q["$next"]}, feedback', 'packed (value, ~index) max per CTA, atomicMax, last CTA publishes and releases the next step of the launch'),
    ]
    sites = ['embed', 'barrier'] + ['qkv', 'barrier', 'attention', 'barrier', 'proj', 'barrier', 'mlp', 'barrier'] + ['logits', 'finish']
    return Lowered(src=src, params=params, scratch=scratch, scratch_floats=scratch_floats, shared_bytes=shared,
                   barriers_per_launch=1 + (4 - int(fuse) - int(fuse_x2) - int(fuse_x3)) * L, plan=plan, sites=sites, counters=32 + max(grid, 1024),
                   block=(nw + 2) * 32, grid=grid, place=rec, packed_bytes=tiles * 512, pack_params=pack_params,
                   dims=dict(dims, B=B, NB=1, tmax=tmax, notes=notes, WG=WG, chunk_tiles=ch, tc=False, ksplit=False, kernel='small', warps=nw,
                             nch=nch, kv_stages=kvst, ring_slots=nslot, fuse_proj=fuse, fuse_exchange=fuse_x, qkv_exchange=fuse_x2, part_exchange=fuse_x3, fuse_base=(fuse_base if fuse else 0), ordered=fixed_sums), roles=roles)

def lower(text, res, axis_max, batch=1, per_token=(), outputs=(), feedback=None, timing=False,
          grid=DEFAULT_SMS, act_lo=None, prompt_len=0, slab_tiles=None, tune=None, row_seq=False):
    """See the module docstring. `res`: name -> (shape, dtype) as the kernel sees them (batched
    where per-token; scalars have shape ()). `axis_max`: bound of the run-time position axis,
    e.g. {'s': tmax}. `grid`: CTAs to place for (one per SM). 't' may be listed in per_token, in
    which case every sequence has its own position (shape (batch,)); a negative position marks a
    sequence that has not started yet. `prompt_len` > 0 adds two kernel parameters after the
    residues, `prompt` (batch, prompt_len) i32 and `plen` (batch,) i32: the feedback then feeds
    prompt[b][t+1] instead of the model's own choice while t + 1 < plen[b], so that prompts (ragged,
    or the reference's tokens for teacher forcing) are consumed without a host round trip. `row_seq=True` makes the rows of
    the batch (cache sequence, position) pairs: the caches may then hold a different number of sequences than the batch has
    rows, a parameter `row_seq` (batch,) i32 follows the residues, and every row attends to its sequence's rows up to its own
    position, those written in the same step included (a dense pass over prompt positions; needs per-sequence positions,
    no feedback, more than eight rows)."""
    env, ext, recv = recognise(text)
    dims = _dims(env, ext)
    D, H, E, F, N, L = dims['D'], dims['H'], dims['E'], dims['F'], dims['N'], dims['L']
    B = int(batch)
    roles = {k: env['$' + k] for k in ROLE_KEYS}
    absent = sorted(k for k, v in roles.items() if v is None)
    roles = {k: (ZEROS if v is None else v) for k, v in roles.items()}
    dims = dict(dims, absent=absent, zeros_len=L * max(3 * D, F))      # (the longest additive parameter: one vector of zeros serves all)
    for role, name in roles.items():
        if name == ZEROS:
            continue
        if name not in res:
            raise NameError(f'residue {name} not supplied')
        if name not in recv:
            raise NameError(f'{name} is used but never received')
    extra = [n for n in res if n not in roles.values()]
    if extra:
        raise ValueError(f'residues the program does not receive: {extra}')
    s_axis = env['$s']
    if s_axis not in axis_max:
        raise ValueError(f'axis_max must bound the run-time axis {s_axis}')
    tmax = int(axis_max[s_axis])
    per_token = set(per_token)
    t_name, x_name = roles['t'], roles['x']
    t_per_token = t_name in per_token

    def want(role, shape, dt):
        if roles[role] == ZEROS:
            return
        got_shape, got_dt = res[roles[role]]
        if tuple(got_shape) != tuple(shape) or got_dt != dt:
            raise ValueError(f'residue {roles[role]}: expected {tuple(shape)} {dt}, got {tuple(got_shape)} {got_dt}')

    wdt = res[roles['wte']][1]
    if wdt != 'f16':
        raise NotImplementedError('weights and the KV cache must be fp16 (f16); fp32 storage is not placed by this backend')
    want('x', (B,), 'i32')
    want('t', (B,) if t_per_token else (), 'i32')
    cpos = int(res[roles['wpe']][0][0])
    want('wte', (N, D), 'f16'); want('wpe', (cpos, D), 'f16')
    for r, shp in (('ln1w', (L, D)), ('ln1b', (L, D)), ('qkvw', (L, D, 3 * D)), ('qkvb', (L, 3 * D)), ('ow', (L, D, D)),
                   ('ob', (L, D)), ('ln2w', (L, D)), ('ln2b', (L, D)), ('fcw', (L, D, F)), ('fcb', (L, F)),
                   ('pw', (L, F, D)), ('pb', (L, D)), ('lnfw', (D,)), ('lnfb', (D,))):
        want(r, shp, 'f16')
    bseq = int(res[roles['keys']][0][0]) if row_seq else B
    if row_seq and (not t_per_token or feedback or B <= 8):
        raise NotImplementedError('row_seq needs per-sequence positions, no feedback and more than eight rows')
    want('keys', (bseq, L, tmax, H, E), 'f16'); want('vals', (bseq, L, tmax, H, E), 'f16')
    for r in ('x', 'keys', 'vals'):
        if roles[r] not in per_token:
            raise NotImplementedError(f'{roles[r]} must be a per-token residue')
    fb = dict(feedback or {})
    if fb and not (fb.get(x_name) == env['$next'] and isinstance(fb.get(t_name), int) and len(fb) == 2):
        raise NotImplementedError(f'feedback must be {{{x_name!r}: {env["$next"]!r}, {t_name!r}: <int>}}')
    for o in outputs:
        if o not in (env['$logit'], env['$next']):
            raise NotImplementedError(f'output {o}: only {env["$logit"]} and {env["$next"]} are kept for the host')

    tune = dict(tune or {})
    if B <= 8 and not tune.get('large_kernel') and act_lo is None and not slab_tiles and not row_seq:
        return _lower_small(env, dims, res, roles, fb, B, tmax, cpos, t_per_token, t_name, prompt_len, timing, grid, tune)

    # rows per slab (8 per batch tile): the operand tiles of a slab live in shared memory next to the
    # weight ring, the K/V tiles and the LayerNorm staging; the largest slab that still leaves three
    # ring slots is taken, larger batches run the contraction phases slab by slab
    KT_D = D // 16
    budget = SMEM_LIMIT - (8192 if timing else 0)      # the timing build keeps its event trace in static shared memory

    # Where the per-CTA LayerNorm is expensive (many rows, or wide rows) each row is normalised once, on one
    # warp of the grid, and the operand tiles pass through global memory (one more barrier per LayerNorm);
    # measured on B200: better from batch 12 at width 768 and at every batch at width 1600.
    tune = dict(tune or {})
    ln_dist = bool(tune.get('ln_dist', B * D >= 12 * 768 or D > 1024))
    # Operand tiles hold the fp16 head and the fp16 remainder of the activations (fp32-accurate products) up to
    # 16 rows (8 at widths above 1024); larger batches keep the head only: half the shared memory per row, twice
    # the rows per slab, logits still within 2e-3 of the reference in the parity tests.
    if act_lo is None:
        act_lo = bool(tune.get('act_lo', B <= 8 or (B <= 16 and D <= 1024)))
    atile = 512 if act_lo else 256

    # K/V tiles in flight per CTA in the attention phase (32 KB each): three where a CTA streams several (sequence,
    # head) items per layer, two (and a deeper weight ring) where it has at most one (measured on B200)
    kvst = int(tune.get('kv_stages', 3 if B * H > grid else 2))

    def smem_fixed(nb):
        return (kvst * (2 * NW * 16 * 128 + 256 + 16) + 32 + KT_D * nb * atile + WN_MAX * nb * atile + NW * nb * 512
                + (3 * D + WN_MAX * 16) * 2 + 16 + 2 * NW * (E + 2) * 4 + 16 + 8 * nb * NW * 8 + B * 4 * (2 if row_seq else 1) + 16 + 8 * 8 + 16 + 32)

    NB = min((B + 7) // 8, 8)
    if slab_tiles:
        NB = min(NB, int(slab_tiles))
    while NB > 1 and (budget - smem_fixed(NB) - 1024) // (CHUNK_TILES * 512 + 16) < 3:
        NB -= 1
    # WIDE groups: output tiles per warp. More than two (tried: six at batch <= 8) gave nothing on B200: the
    # contractions of a small batch are bound by the latency of their few dependent steps, not by issue slots.
    tpw = int(tune.get('tpw', 2))
    wg = tpw * NW
    ch = max(CHUNK_TILES, wg)
    # Large batches: the MLP projection, which combines partial sums with fp32 atomics, gets few, deep slices of the
    # fold (a 6-way instead of a 148-way sum: its atomics cost 1,900 cycles per group of 16 output tiles and slab),
    # at the price of one more grid barrier per layer and the GELU output passing through global memory; possible
    # where a slice of the MLP fold fits the operand tiles. Measured on B200: batch 64, 1,037 -> 938 us per step;
    # 256 ragged sequences, 3,146 -> 2,735. (The same placement for the attention projection was slower: its
    # operand is merged from the attention partials element by element, eight times more of them per CTA.)
    _groups = math.ceil((D // 16) / 2)
    _nk = math.ceil((F // 16) / max(1, min(F // 16, grid // _groups))) if _groups <= grid else 1 << 30
    ksplit = bool(tune.get('ksplit', B >= 32) and _nk <= KT_D and _groups <= grid)
    # Tensor cores (tcgen05, accumulators in tensor memory) where the contractions are dense: 64 sequences and more.
    # The logits as tiles of 128 vocabulary rows x 64 sequences (the fp16 operand of 64 sequences, 64 x D x 2 bytes,
    # takes the place of the K/V stages, a 128 x 64 tile of the table one ring slot). The four layer contractions with
    # the sequences as the rows of the product: units of a block of `tcl_rb` sequences (64; 32 measured slower at 64 sequences)
    # x `tcl_nw` output columns (32) x the D / 64 k-blocks of a fold of width D (the MLP projection in F / D parts,
    # combined with atomics), from a packed weight image; where the operand of a row block fits the K/V stages and a
    # unit's weights a whole number of ring slots (which divides the slots a logits tile row takes, so that a unit never
    # wraps around the ring). Measured on B200 against units of 128 output columns x 64 sequences
    # (18 to 24 units per phase at 64 sequences, the other CTAs waiting): see the profile of batch 64.
    tc = bool(tune.get('tc', True) and B >= 64 and ln_dist and not act_lo and D % 64 == 0
              and 64 * D * 2 <= kvst * 2 * NW * 16 * 128 and ch * 512 == 16384)
    kbd, kbf = D // 64, F // 64
    tcl_nw = int(tune.get('tcl_nw', 32))
    tcl_rb = int(tune.get('tcl_rb', 64))
    if tcl_nw not in (16, 32) or tcl_rb not in (32, 64):
        raise ValueError('tcl_nw must be 16 or 32, tcl_rb 32 or 64')
    tcl_spu = -(-(tcl_nw * 128 * kbd) // 16384)
    # (the product reads 64 rows from the start of every k-block of the operand: the last one reaches past the stages,
    # into the operand tiles of the mma.sync path, which this mode leaves unused)
    kv_bytes = kvst * 2 * NW * 16 * 128
    tcl = bool(tc and tune.get('tc_layers', True) and D % tcl_nw == 0 and F % D == 0 and kbd % tcl_spu == 0 and kbd * tcl_rb * 128 <= kv_bytes
               and (kbd - 1) * tcl_rb * 128 + 8192 <= kv_bytes + KT_D * atile and B * 4 <= KT_D * atile and ksplit)
    rec, tiles, notes = place_step(dims, grid, ksplit)
    if tcl:
        NB = 1          # the mma.sync operand tiles are not used: their shared memory goes to the weight ring

    # global scratch (floats): host-visible values first, then the kernel's own vectors
    def up(v, a=64):
        return (v + a - 1) // a * a
    off_logit, off_next = 0, up(B * N)
    off_z = up(off_next + B)
    off_q = off_z + 3 * up(B * D)
    # position chunks per (sequence, head) in the attention phase: rounds of the grid x (positions per chunk
    # + the fixed cost of an item, about one tile of 128 positions), at a typical context of tmax / 2
    def att_cost(k):
        return math.ceil(B * H * k / grid) * (max(tmax // 2, 1) / k + 192)
    nch = min(range(1, 17), key=lambda k: (att_cost(k), k))
    tune = dict(tune or {})
    nch = int(tune.get('nch', nch))
    # With more (sequence, head) pairs than CTAs and one chunk each, the pairs left over after whole rounds of the
    # grid are split into position chunks, so that the last round costs every CTA a fraction of an item. Only
    # where a chunk still is a full tile of positions at a typical context (measured: no gain at batch 64 with
    # contexts of 512-1024, a loss of 3 % with contexts of 128-384).
    tail_bh, ts = B * H, 1
    if tcl and nch != 1:
        raise NotImplementedError('tensor-core layer contractions take the attention output of whole (sequence, head) items')
    if nch == 1 and B * H > grid and (B * H) % grid and tune.get('tail_split', True) and not tcl:
        left = (B * H) % grid
        want = tune.get('tail_split', True)
        ts = min(grid // left, 8, max(tmax // 2, 1) // 128) if want is True else min(grid // left, int(want))
        if ts > 1:
            tail_bh = B * H - left
        else:
            ts = 1
    att_items = tail_bh * nch + (B * H - tail_bh) * ts
    off_part = off_q + up(B * D)
    off_actg = off_part + up(att_items * (E + 2))
    off_best = off_actg + (up(((B + 8 * NB - 1) // (8 * NB)) * KT_D * NB * atile // 4) if ln_dist else 0)
    off_tc = off_best + up(2 * B)
    off_gg = off_tc + (up(((B + 63) // 64) * 64 * D * 2 // 4) if tc else 0)
    # V_KSPLIT: the GELU outputs as operand tiles, per slab [fold tile of F][batch tile]; with tensor-core layer
    # contractions as fp16 K-major swizzled rows per slab of 64 sequences, like the attention output behind them
    tc_slabs = (B + 63) // 64
    off_og = off_gg + ((up(tc_slabs * 64 * F * 2 // 4) if tcl else up(((B + 8 * NB - 1) // (8 * NB)) * (F // 16) * NB * atile // 4)) if ksplit else 0)
    scratch_floats = off_og + (up(tc_slabs * 64 * D * 2 // 4) if tcl else 0)
    scratch = {env['$logit']: (off_logit, ('bt', env['$n']), (B, N)), env['$next']: (off_next, ('bt',), (B,))}

    fixed = smem_fixed(NB)
    nslot = (budget - fixed - 1024) // (ch * 512 + 16)
    if nslot < 2:
        raise NotImplementedError('model too wide for the shared-memory budget at this batch')
    nslot = min(nslot, 16)
    if tcl:
        nslot = nslot // tcl_spu * tcl_spu          # a unit's weights take tcl_spu consecutive slots and never wrap
        if nslot < tcl_spu:
            raise NotImplementedError('the weights of a tensor-core unit do not fit the ring')
    shared = fixed + nslot * (ch * 512 + 16) + 512

    def f32(v):
        return repr(float(np.float32(v))) + 'f'
    scale = dims['scale']
    defs = dict(V_NW=NW, V_B=B, V_NB=NB, V_L=L, V_D=D, V_H=H, V_E=E, V_F=F, V_N=N, V_TMAX=tmax, V_CPOS=cpos,
                V_EPS=f32(dims['eps']), V_SCALE=f32(scale), V_SCALE_IS_POW2=int(math.frexp(scale)[0] == 0.5), V_GELU_A=f32(dims['gelu'][0]), V_GELU_B=f32(dims['gelu'][1]),
                V_GELU_C=f32(dims['gelu'][2]), V_NSLOT=nslot, V_CH=ch, V_TPW=tpw, V_KVST=kvst, V_ACT_LO=int(bool(act_lo)),
                V_TSTRIDE=int(t_per_token), V_FEEDBACK=int(bool(fb)), V_TSTEP=int(fb.get(t_name, 0)),
                V_TIMING=int(timing), V_PLEN=int(prompt_len) if fb else 0, V_OFF_LOGIT=off_logit, V_OFF_NEXT=off_next, V_OFF_Z=off_z, V_OFF_Q=off_q,
                V_MAXGRID=grid, V_LN_DIST=int(ln_dist), V_OFF_ACTG=off_actg, V_OFF_PART=off_part, V_OFF_BEST=off_best, V_TC=int(tc), V_OFF_TC=off_tc, V_ROWSEQ=int(bool(row_seq)), V_BSEQ=bseq, V_TCL=int(tcl), V_TCL_NW=tcl_nw, V_TCL_RB=tcl_rb, V_ATT_SNAKE=int(tune.get('att_snake', 1)), V_OFF_OG=off_og, V_KSPLIT=int(ksplit), V_OFF_GG=off_gg, V_NCH=nch, V_TAIL_BH=tail_bh, V_TS=ts, V_WAIT_NS=f"{int(tune.get('wait_ns', 500_000_000))}ull")
    head = ''.join(f'#define {k} {v}\n' for k, v in defs.items())

    params, pack_params, tail = _entry_points(res, roles, fb, prompt_len, row_seq)
    src = head + COMMON_TEXT.read_text(encoding='utf-8') + KERNEL_TEXT.read_text(encoding='utf-8') + tail

    q = env
    ln_how = ('each row normalised once on one warp of the grid, operand tiles through global memory (+1 barrier)' if ln_dist
              else 'every CTA recomputes, one warp per row held in registers, into mma operand tiles')
    att_items_txt = (f'{tail_bh} whole (sequence, head) items, the other {B * H - tail_bh} in {ts} position chunks' if ts > 1
                     else f'one item per (sequence, head, 1/{nch} of the positions)')
    plan = [
        (f'{q["$z0"]} (embed)', 'grid-stride, then barrier'),
        (f'{q["$m1"]}, {q["$v1"]}, {q["$a"]} (LN1)', ln_how),
        (f'{q["$qkv"]} + emits', f'NARROW: whole fold, {min(rec[:, 3])}-{max(rec[:, 3])} output tiles per CTA; bias, q, K/V emit in the epilogue'),
        (f'{q["$sc"]}, {q["$mx"]}, {q["$ex"]}, {q["$w"]}, {q["$o"]} (attention)',
         f'{att_items_txt}, dealt round-robin over the CTAs; K/V tiles by TMA ({kvst} stages), online softmax in registers, merged by the projection'),
        (f'{q["$oo"]}, {q["$z1"]}', f'WIDE: {notes["proj_units"]} units of up to {WG} output tiles x {notes["proj_nk"]} fold tiles, fp32 atomics'),
        (f'{q["$m2"]}, {q["$v2"]}, {q["$b"]} (LN2)', ln_how),
        (f'{q["$u"]}, {q["$g"]}', f'NARROW: {min(rec[:, 9])}-{max(rec[:, 9])} f tiles per CTA, GELU in the epilogue, result '
                                  + ('through global memory as operand tiles (+1 barrier)' if ksplit else 'stays in shared memory')),
        (f'{q["$z2"]}', (f'NARROW: two output tiles x {notes["p2_nk"]} fold tiles per CTA, fp32 atomics' if ksplit
                         else 'WIDE over the CTA\'s own f tiles, fp32 atomics')),
        (f'{q["$m3"]}, {q["$v3"]}, {q["$c"]} (LNf)', ln_how),
        (f'{q["$logit"]}', ('tcgen05.mma tiles of 128 vocabulary rows x 64 sequences, accumulators in tensor memory, ' if tc else 'WIDE over the whole fold, ')
                           + f'{min(rec[:, 11])}-{max(rec[:, 11])} vocabulary tiles per CTA'),
        (f'{q["$best"]}, {q["$next"]}, feedback', 'packed (value, ~index) max per CTA, atomicMax, last CTA publishes and releases the next step of the launch'),
    ]
    sites = ['embed', 'barrier'] + ['qkv', 'barrier', 'attention', 'barrier', 'proj', 'barrier', 'mlp', 'barrier'] \
        + ['logits', 'finish']
    low = Lowered(src=src, params=params, scratch=scratch, scratch_floats=scratch_floats, shared_bytes=shared,
                  barriers_per_launch=1 + (4 + int(ksplit)) * L + ((2 * L + 1) if ln_dist else 0), plan=plan, sites=sites, counters=32 + max(grid, 1024),
                  block=(NW + 1) * 32, grid=grid, place=rec, pack_params=pack_params,
                  packed_bytes=(L * (3 * D + D + F + D * (F // D)) // tcl_nw * (tcl_nw * 128 * kbd)) if tcl else tiles * 512,
                  dims=dict(dims, B=B, NB=NB, tmax=tmax, notes=notes, WG=wg, chunk_tiles=ch, tc=tc, ksplit=ksplit, tcl=tcl,
                            tcl_unit=(tcl_rb, tcl_nw), kernel='large'), roles=roles)
    return low
