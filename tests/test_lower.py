"""Recognition and placement (vesta_gpu_b200/lower.py), on the CPU."""
import numpy as np
import pytest

from vesta_gpu_b200 import lower as lw
from vesta_gpu_b200.build import lower_for, residue_spec
from vesta_gpu_b200.program_text import decode_program
from vesta_gpu_b200.shapes import GPT2_SMALL, GPT2_XL, TINY, TINY3


def stream_tiles(rec, dims, cta):
    """tiles of one CTA's stream as (kind, layer, j tile, k tile), in stream order: the index
    arithmetic of pack_narrow / pack_wide in csrc/step_kernel.cuh restated"""
    D, F, N, L = dims['D'], dims['F'], dims['N'], dims['L']
    KT_D, JT_D = D // 16, D // 16
    base, layer, qj0, qnj, pj0, pnj, pk0, pnk, fj0, fnj, lj0, lnj = [int(v) for v in rec[cta][:12]]
    WG = dims['WG']                                  # output tiles per WIDE group of this lowering

    def narrow(kind, l, j0, nj, kt, k0=0):
        return [(kind, l, j0 + i % nj, k0 + i // nj) for i in range(nj * kt)]

    def wide(kind, l, j0, nj, k0, nk):
        out = []
        for i in range(nj * nk):
            grp = i // (WG * nk)
            width = min(WG, nj - grp * WG)
            r = i - grp * WG * nk
            out.append((kind, l, j0 + grp * WG + r % width, k0 + r // width))
        return out
    tiles = []
    for l in range(L):
        if dims['ksplit']:                           # the MLP projection as (two output tiles x a slice of the fold)
            qj0_, qnj_, qk0_, qnk_ = [int(v) for v in rec[cta][12:16]]
            seg = narrow('qkv', l, qj0, qnj, KT_D) + wide('proj', l, pj0, pnj, pk0, pnk) \
                + narrow('fc', l, fj0, fnj, KT_D) + narrow('p2', l, qj0_, qnj_, qnk_, qk0_)
        elif dims.get('fuse_proj'):                  # the attention projection is applied per head by the attention items
            seg = narrow('qkv', l, qj0, qnj, KT_D) + narrow('fc', l, fj0, fnj, KT_D) + wide('p2', l, 0, JT_D, fj0, fnj)
        else:
            seg = narrow('qkv', l, qj0, qnj, KT_D) + wide('proj', l, pj0, pnj, pk0, pnk) \
                + narrow('fc', l, fj0, fnj, KT_D) + wide('p2', l, 0, JT_D, fj0, fnj)
        assert len(seg) == layer
        tiles += seg
    tiles += wide('logit', 0, lj0, lnj, 0, KT_D)
    return base, tiles


@pytest.mark.parametrize('sh,batch,grid', [(GPT2_SMALL, 1, 148), (GPT2_SMALL, 8, 148), (TINY, 3, 148), (TINY3, 2, 148),
                                           (GPT2_XL, 1, 148), (GPT2_SMALL, 8, 132), (TINY, 1, 7),
                                           (GPT2_SMALL, 64, 148), (TINY3, 40, 148), (GPT2_SMALL, 256, 132)])
def test_every_weight_tile_exactly_once(sh, batch, grid):
    low = lower_for(sh, batch, 64, grid=grid, tune=dict(ksplit=True, tc_layers=False) if batch >= 40 else None)      # (the mma.sync streams)
    assert low.dims['ksplit'] == (batch >= 40)
    dims = low.dims
    D, F, N, L = dims['D'], dims['F'], dims['N'], dims['L']
    want = {'qkv': (3 * D // 16, D // 16), 'proj': (D // 16, D // 16), 'fc': (F // 16, D // 16),
            'p2': (D // 16, F // 16), 'logit': ((N + 15) // 16, D // 16)}
    seen = {k: np.zeros((L if k != 'logit' else 1,) + v, np.int32) for k, v in want.items()}
    cursor = 0
    for c in range(grid):
        base, tiles = stream_tiles(low.place, dims, c)
        assert base == cursor                       # streams are laid end to end
        cursor += len(tiles)
        for kind, l, j, k in tiles:
            seen[kind][l, j, k] += 1
    if dims.get('fuse_proj'):
        # behind the per-CTA streams: per layer and head the head's 64 rows of the projection, output tile major
        assert cursor == dims['fuse_base']
        fus = dims['E'] // 16
        for l in range(L):
            for h in range(dims['H']):
                for i in range((D // 16) * fus):
                    seen['proj'][l, i // fus, h * fus + i % fus] += 1
                    cursor += 1
    assert cursor * 512 == low.packed_bytes
    for k, v in seen.items():
        assert v.min() == 1 and v.max() == 1, k
    # every output tile of the projection has exactly one CTA that starts at fold tile 0, NARROW widths fit
    assert low.place[:, 3].max() <= lw.WN_MAX and low.place[:, 9].max() <= lw.WN_MAX


def test_tensor_core_weight_image_covers_every_weight_once():
    """64 sequences and more: the packed image of the layer weights is a list of (fold part, output block) blocks of
    V_TCL_NW output columns x D fold indices per layer and contraction (pack_body / tcl_* in csrc/step_kernel.cuh
    restated); the runs of units of the CTAs cover every (row block, fold part, output block) exactly once, the
    operand of a row block fits the K/V stages and a unit's weights a whole number of ring slots"""
    for sh, B, tune in ((GPT2_SMALL, 64, {}), (GPT2_SMALL, 256, {}), (TINY, 130, {}), (TINY, 130, dict(tcl_nw=16, tcl_rb=32))):
        low = lower_for(sh, B, 64, tune=dict(tune, ln_dist=True))
        assert low.dims['tcl'] and low.dims['tc'] and low.dims['ksplit']
        D, F, L = sh.D, sh.F, sh.L
        rb_rows, nw = low.dims['tcl_unit']
        assert rb_rows == define(low, 'V_TCL_RB') and nw == define(low, 'V_TCL_NW')
        assert rb_rows == tune.get('tcl_rb', 64)
        uk = D // 64
        ub = nw * 128 * uk
        nfb = {'qkv': 3 * D // nw, 'proj': D // nw, 'fc': F // nw, 'p2': D // nw}
        nks = {'qkv': 1, 'proj': 1, 'fc': 1, 'p2': F // D}
        assert low.packed_bytes == L * sum(nfb[k] * nks[k] for k in nfb) * ub == 2 * L * (D * 3 * D + D * D + 2 * D * F)   # every weight element once
        slot = define(low, 'V_CH') * 512
        spu = -(-ub // slot)
        assert define(low, 'V_NSLOT') % spu == 0 and define(low, 'V_NSLOT') >= spu
        assert uk * rb_rows * 128 <= define(low, 'V_KVST') * 32768                  # the operand of a row block fits the K/V stages
        nrb = -(-B // rb_rows)
        for k in nfb:
            n = nrb * nks[k] * nfb[k]
            seen = np.zeros((nrb, nks[k], nfb[k]), np.int32)
            for cta in range(low.grid):
                for u in range(cta * n // low.grid, (cta + 1) * n // low.grid):
                    r, rest = divmod(u, nks[k] * nfb[k])
                    s_, f_ = divmod(rest, nfb[k])
                    seen[r, s_, f_] += 1
            assert seen.min() == 1 and seen.max() == 1
    # 64 sequences at GPT-2 small: 72 QKV units of 64 sequences x 32 output columns (18 of 128 x 64 before)
    low = lower_for(GPT2_SMALL, 64, 64, tune=dict(ln_dist=True))
    assert -(-64 // low.dims['tcl_unit'][0]) * (3 * 768 // low.dims['tcl_unit'][1]) == 72


def test_every_phase_has_the_smallest_possible_largest_share():
    """the phases are separated by grid barriers, so a phase costs what its busiest CTA has: no CTA holds more than
    ceil(tiles / CTAs) output tiles of the QKV, FC and logits contractions, and one projection unit at most"""
    for sh, b in ((GPT2_SMALL, 8), (GPT2_XL, 1), (TINY3, 2)):
        low = lower_for(sh, b, 64)
        r, d, G = low.place, low.dims, low.grid
        ceil = lambda a: -(-a // G)
        assert r[:, 3].max() == ceil(3 * d['D'] // 16) and r[:, 3].sum() == 3 * d['D'] // 16
        assert r[:, 9].max() == ceil(d['F'] // 16) and r[:, 9].sum() == d['F'] // 16
        jt_n = (d['N'] + 15) // 16
        assert r[:, 11].max() == ceil(jt_n) and r[:, 11].min() >= jt_n // G and r[:, 11].sum() == jt_n
    n = lower_for(GPT2_SMALL, 8, 384).dims['notes']
    assert n['tiles_max'] / n['tiles_mean'] < 1.3        # the bytes per CTA and step follow from that, within 30 %


def test_lowered_fields_match_reference_contract():
    """vesta/lower.py:69-79: src, params, scratch, scratch_floats, shared_bytes, barriers_per_launch, plan, sites, counters"""
    low = lower_for(GPT2_SMALL, 8, 384)
    names = [p[0] for p in low.params]
    assert names == ['x', 't', 'wte', 'wpe', 'ln1w', 'ln1b', 'qkvw', 'qkvb', 'ow', 'ob', 'ln2w', 'ln2b', 'fcw', 'fcb',
                     'pw', 'pb', 'lnfw', 'lnfb', 'keys', 'vals']
    emitted = {p[0] for p in low.params if p[2]}
    assert emitted == {'x', 't', 'keys', 'vals'}
    off, axes, shape = low.scratch['logit']
    assert shape == (8, 50257) and off == 0
    off2, _, shape2 = low.scratch['next']
    assert shape2 == (8,) and off2 >= 8 * 50257 and low.scratch_floats > off2 + 8
    assert low.shared_bytes <= 227 * 1024
    assert low.barriers_per_launch == 1 + 2 * 12          # two per layer (query / K / V and the heads' outputs travel as tagged values between the CTAs that need them); the reference needs 113 at batch 8
    assert lower_for(GPT2_SMALL, 8, 384, tune=dict(qkv_exchange=False)).barriers_per_launch == 1 + 3 * 12
    assert lower_for(GPT2_SMALL, 8, 384, tune=dict(fuse_proj=False, qkv_exchange=False)).barriers_per_launch == 1 + 4 * 12
    assert lower_for(GPT2_SMALL, 1, 384).barriers_per_launch == 1 + 2 * 12             # one sequence: the pairs are cut into chunks, the projection keeps its phase but polls the chunks' results
    assert lower_for(GPT2_SMALL, 1, 384, tune=dict(part_exchange=False)).barriers_per_launch == 1 + 3 * 12
    assert 'vesta_step' in low.src and 'vesta_pack' in low.src and low.counters >= 64
    assert len(low.plan) >= 8 and all(len(p) == 2 for p in low.plan)
    no_fb = lower_for(GPT2_SMALL, 1, 64, feedback=False)
    assert {p[0] for p in no_fb.params if p[2]} == {'keys', 'vals'}


def test_constants_read_from_the_program():
    low = lower_for(GPT2_XL, 1, 64)
    d = low.dims
    assert (d['L'], d['D'], d['H'], d['F'], d['N']) == (48, 1600, 25, 6400, 50257)
    assert d['eps'] == 1e-5 and d['scale'] == 8.0 and d['gelu'] == (0.5, 0.7978845608028654, 0.044715)
    text = decode_program(TINY, eps=0.001)
    spec = residue_spec(TINY, 1, 16)
    low = lw.lower(text, spec, {'s': 16}, batch=1, per_token=('x', 'keys', 'vals'), outputs=('logit', 'next'))
    assert low.dims['eps'] == 0.001 and '#define V_EPS 0.001' in low.src


def mutate(text, old, new):
    assert old in text
    return text.replace(old, new, 1)


@pytest.mark.parametrize('old,new', [
    ('tanh(', 'exp('),                                   # another activation
    ('/ 8', '* 8'),                                      # scores multiplied instead of divided
    ('z1[d] = z[d] + oo[d] + ob[l, d]', 'z1[d] = oo[d] + ob[l, d]'),      # no residual
    ('fold max s: sc[h, s]', 'fold min s: sc[h, s]'),
    ('next = fold min n:', 'next = fold max n:'),        # ties to the highest id
    ('axis j = 384', 'axis j = 400'),                    # QKV not three widths
    ('    q[h, e] = qkv[h * 64 + e]\n', ''),             # a statement missing
])
def test_programs_outside_the_family_are_refused(old, new):
    text = mutate(decode_program(TINY), old, new)
    with pytest.raises(NotImplementedError):
        lw.lower(text, residue_spec(TINY, 1, 16), {'s': 16}, batch=1, per_token=('x', 'keys', 'vals'))


def test_residue_checks():
    text = decode_program(TINY)
    spec = residue_spec(TINY, 2, 16)
    with pytest.raises(ValueError):
        lw.lower(text, dict(spec, wte=((TINY.N, TINY.D + 16), 'f16')), {'s': 16}, batch=2, per_token=('x', 'keys', 'vals'))
    with pytest.raises(NameError):
        lw.lower(text, {k: v for k, v in spec.items() if k != 'pb'}, {'s': 16}, batch=2, per_token=('x', 'keys', 'vals'))
    with pytest.raises(NotImplementedError):
        lw.lower(text, dict(spec, wte=((TINY.N, TINY.D), 'f32')), {'s': 16}, batch=2, per_token=('x', 'keys', 'vals'))
    with pytest.raises(ValueError):
        lw.lower(text, spec, {}, batch=2, per_token=('x', 'keys', 'vals'))
    with pytest.raises(NotImplementedError):
        lw.lower(text, spec, {'s': 16}, batch=2, per_token=('x', 'keys', 'vals'), feedback={'x': 'best', 't': 1})


def test_renamed_program_is_recognised():
    """names are read from the program, not assumed"""
    text = decode_program(TINY).replace('qkv', 'proj3').replace('zL', 'out_state').replace('sc[', 'score[').replace('sc[h, s]', 'score[h, s]')
    spec = residue_spec(TINY, 1, 16)
    spec = {k.replace('qkv', 'proj3'): v for k, v in spec.items()}
    low = lw.lower(text, spec, {'s': 16}, batch=1, per_token=('x', 'keys', 'vals'), outputs=('logit', 'next'))
    assert low.roles['qkvw'] == 'proj3w' and 'R_proj3w' in low.src


@pytest.mark.parametrize('without', [('qkvb',), ('ln1b', 'ln2b', 'lnfb'), ('ob', 'pb'), ('ln1b', 'qkvb', 'ob', 'ln2b', 'fcb', 'pb', 'lnfb')])
@pytest.mark.parametrize('batch', [1, 70])
def test_programs_without_shifts_or_biases_are_placed(without, batch):
    """the additive parameters may be absent from a program (a model without biases, LayerNorms without shift): the
    statements are matched without their last term, the residues are neither received nor bound, and the kernel gets one
    vector of zeros in their place; the interpreter of the reference runs such a program as it stands"""
    text = decode_program(TINY, without=without)
    assert all(f'residue {n}[' not in text for n in without)
    spec = {k: v for k, v in residue_spec(TINY, batch, 16).items() if k not in without}
    low = lw.lower(text, spec, {'s': 16}, batch=batch, per_token=('x', 'keys', 'vals'), outputs=('logit', 'next'),
                   tune=dict(ln_dist=True) if batch > 8 else None)
    names = [p[0] for p in low.params]
    assert names[-1] == '_zeros' and not set(without) & set(names)
    assert low.dims['absent'] == sorted(without) and low.dims['zeros_len'] >= TINY.L * max(3 * TINY.D, TINY.F)
    assert all(low.roles[n] == '_zeros' for n in without) and 'X_zeros' in low.src
    # a residue that is supplied but not received is still an error; a multiplicative parameter cannot be left out
    with pytest.raises(ValueError):
        lw.lower(text, residue_spec(TINY, batch, 16), {'s': 16}, batch=batch, per_token=('x', 'keys', 'vals'))
    with pytest.raises(NotImplementedError):
        lw.lower(decode_program(TINY).replace(' * ln1w[l, d]', ''), residue_spec(TINY, 1, 16), {'s': 16}, batch=1, per_token=('x', 'keys', 'vals'))


def test_per_sequence_positions():
    low = lower_for(TINY, 4, 32, per_sequence_t=True)
    assert '#define V_TSTRIDE 1' in low.src
    assert dict((p[0], p[1]) for p in low.params)['t'] == 'i32'


def test_slabs_and_device_side_prompts():
    low = lower_for(GPT2_SMALL, 64, 1024, tune=dict(tc_layers=False))
    assert low.dims['NB'] == 4 and '#define V_LN_DIST 1' in low.src        # mma.sync contractions: 32 rows per slab, rows normalised once
    low = lower_for(GPT2_SMALL, 64, 1024)
    assert low.dims['tcl'] and low.dims['NB'] == 1 and '#define V_LN_DIST 1' in low.src      # tensor-core contractions: no operand tiles in shared memory
    assert low.shared_bytes <= 227 * 1024
    low = lower_for(TINY, 20, 16, slab_tiles=1)
    assert low.dims['NB'] == 1
    low = lower_for(TINY, 4, 16, per_sequence_t=True, prompt_len=9)
    assert [p[0] for p in low.params][-2:] == ['prompt', 'plen'] and '#define V_PLEN 9' in low.src
    low = lower_for(TINY, 4, 16, feedback=False, prompt_len=9)            # nothing to feed back into
    assert [p[0] for p in low.params][-1] == 'vals' and '#define V_PLEN 0' in low.src


def define(low, name):
    for line in low.src.split('\n'):
        if line.startswith(f'#define {name} '):
            return int(line.split()[2])
    raise KeyError(name)


def test_tensor_core_logits_are_chosen_where_the_contraction_is_dense():
    """64 sequences and more, fp16-head operands, an operand of 64 sequences that fits the K/V stages"""
    assert define(lower_for(GPT2_SMALL, 64, 1025), 'V_TC') == 1
    assert define(lower_for(GPT2_SMALL, 256, 640), 'V_TC') == 1
    assert define(lower_for(GPT2_SMALL, 63, 64), 'V_TC') == 0
    assert lower_for(GPT2_SMALL, 8, 384).dims['kernel'] == 'small' and not lower_for(GPT2_SMALL, 8, 384).dims['tc']
    assert define(lower_for(GPT2_SMALL, 8, 384, tune=dict(large_kernel=True)), 'V_TC') == 0
    assert define(lower_for(GPT2_XL, 64, 64), 'V_TC') == 0              # 64 x 1600 halves exceed the stages
    assert define(lower_for(GPT2_SMALL, 64, 64, tune=dict(tc=False)), 'V_TC') == 0
    low = lower_for(GPT2_SMALL, 64, 1025)
    assert low.scratch_floats * 4 >= define(low, 'V_OFF_TC') * 4 + 64 * 768 * 2


def test_attention_items_cover_every_sequence_head_and_position():
    """the item arithmetic of the attention phase (att_item / att_load_item in csrc/step_kernel.cuh) restated: whole
    rounds of one item per (sequence, head), then the leftover pairs split into position chunks"""
    for sh, B, tmax, tune in ((GPT2_SMALL, 64, 1025, dict(tc_layers=False)), (GPT2_SMALL, 1, 384, dict(large_kernel=True)), (TINY3, 60, 6, dict(tail_split=4)),
                              (GPT2_SMALL, 64, 400, dict(tc_layers=False)), (GPT2_SMALL, 64, 1025, None)):
        low = lower_for(sh, B, tmax, tune=tune)
        nch, tail_bh, ts, H = define(low, 'V_NCH'), define(low, 'V_TAIL_BH'), define(low, 'V_TS'), low.dims['H']
        items = tail_bh * nch + (B * H - tail_bh) * ts
        for n in (1, 5, tmax):                                           # attended positions of every sequence
            seen = np.zeros((B * H, n), np.int32)
            for it in range(items):
                if it < tail_bh * nch:
                    bh, ch, k = it // nch, it % nch, nch
                else:
                    j = it - tail_bh * nch
                    bh, ch, k = tail_bh + j // ts, j % ts, ts
                cs = (max(n, 1) + k - 1) // k
                seen[bh, ch * cs: min(n, (ch + 1) * cs)] += 1
            assert seen.min() == 1 and seen.max() == 1
        if sh is GPT2_SMALL and B == 64 and tmax == 1025 and tune:
            assert ts == 4 and tail_bh == 740 and items <= 6 * 148        # five whole rounds and one of quarter items
        if tune is None:
            assert ts == 1 and nch == 1 and low.dims['tcl']              # tensor-core contractions take whole (sequence, head) items


def small_tile_list(low, cta, pos):
    """build_tile_list of csrc/step_small.cuh restated: the K/V tiles of one CTA for the positions `pos` of the sequences"""
    nch, H, kvst, maxtl, grid = define(low, 'V_NCH'), low.dims['H'], define(low, 'V_KVST'), define(low, 'V_MAXTL'), low.grid
    out, live = [], 0
    for it in range(cta, len(pos) * H * nch, grid):
        bh, ch = divmod(it, nch)
        b, h = divmod(bh, H)
        npos = pos[b] + 1
        cs = (max(npos, 1) + nch - 1) // nch
        s, hi = ch * cs, min(npos, (ch + 1) * cs)
        if hi <= s:
            out.append(dict(b=b, h=h, s=0, cnt=0, last=True, patch=False, item=it))
            continue
        while s < hi:
            cnt = min(128, hi - s)
            out.append(dict(b=b, h=h, s=s, cnt=cnt, last=s + 128 >= hi, patch=live < kvst and s <= pos[b] < s + cnt, item=it))
            live += 1
            s += 128
    assert len(out) <= maxtl, (len(out), maxtl)
    return out


def test_small_kernel_tile_lists_cover_every_sequence_head_and_position():
    """at most eight sequences: every (sequence, head, position) is in exactly one tile of one CTA, every item ends with a
    `last` tile, the list fits the space the lowering reserved, and the tile that holds the current position is marked
    for patching whenever it can be requested before the barrier (among the first V_KVST tiles of its CTA)"""
    for sh, B, tmax, pos in ((GPT2_SMALL, 8, 385, [384] * 8), (GPT2_SMALL, 8, 385, [0, 5, 127, 128, 129, 300, 383, -3]),
                             (GPT2_SMALL, 1, 1024, [1023]), (GPT2_XL, 1, 385, [200]), (TINY3, 5, 9, [8, 0, 3, -1, 4]),
                             (GPT2_XL, 8, 1024, [1023] * 8)):
        low = lower_for(sh, B, tmax, per_sequence_t=True)
        assert low.dims['kernel'] == 'small'
        seen = [np.zeros((sh.H, max(p + 1, 0)), np.int32) for p in pos]
        items = set()
        for cta in range(low.grid):
            tl = small_tile_list(low, cta, pos)
            for k, e in enumerate(tl):
                seen[e['b']][e['h'], e['s']: e['s'] + e['cnt']] += 1
                if e['last']:
                    assert e['item'] not in items
                    items.add(e['item'])
                early = sum(1 for f in tl[:k] if f['cnt']) < define(low, 'V_KVST')
                holds = e['cnt'] and e['s'] <= pos[e['b']] < e['s'] + e['cnt']
                assert e['patch'] == bool(early and holds)
        assert all(v.size == 0 or (v.min() == 1 and v.max() == 1) for v in seen)
        assert items == set(range(B * sh.H * define(low, 'V_NCH')))
        assert low.shared_bytes <= 227 * 1024


def test_small_division_by_reciprocal_is_exact():
    """qdiv in csrc/step_kernel.cuh: a / w as trunc((a + 0.5) * (1 / w)) in fp32 with a reciprocal that is off by up to
    two ulps, for every a < 4096 and w <= 64 (the kernel's operands: tiles per chunk, warps, fold tiles per CTA)"""
    a = np.arange(0, 4096, dtype=np.int32)
    for w in range(1, 65):
        r = np.float32(1.0) / np.float32(w)
        lo = np.nextafter(np.nextafter(r, np.float32(0)), np.float32(0))
        hi = np.nextafter(np.nextafter(r, np.float32(2)), np.float32(2))
        for rr in (lo, r, hi):
            q = ((a.astype(np.float32) + np.float32(0.5)) * rr).astype(np.int32)
            assert np.array_equal(q, a // w), w


def test_exchanges_between_ctas_are_chosen_where_every_cta_has_at_most_one_item():
    """at most eight sequences: where the attention items are no more than the CTAs, the values a phase needs from a few
    other CTAs travel as tagged 8-byte pairs (no CTA then waits for a value whose producer waits): query / K / V rows to
    the attention items; the items' outputs inside a head (one chunk per pair) or the chunks' partial results to the
    projection phase (several chunks); two grid barriers per layer are left. The buffers lie 8-byte aligned in the
    scratch area, behind the partial results."""
    for sh, B, tmax in ((GPT2_SMALL, 8, 384), (GPT2_SMALL, 1, 384), (GPT2_SMALL, 2, 384), (GPT2_XL, 1, 384), (TINY, 3, 16)):
        low = lower_for(sh, B, tmax)
        d = low.dims
        assert d['kernel'] == 'small' and d['qkv_exchange']
        assert d['fuse_exchange'] == bool(d['fuse_proj']) and d['part_exchange'] == (not d['fuse_proj'])
        assert B * sh.H * d['nch'] <= low.grid
        assert low.barriers_per_launch == 1 + 2 * sh.L
        off_x, off_part, off_best = define(low, 'V_OFF_X'), define(low, 'V_OFF_PART'), define(low, 'V_OFF_BEST')
        assert off_x % 2 == 0 and off_part % 2 == 0
        pairs = sh.H * B * sh.E * (int(d['fuse_exchange']) + 3)
        assert off_best - off_x >= 2 * pairs and off_x - off_part >= B * sh.H * d['nch'] * (sh.E + 2) * (2 if d['part_exchange'] else 1)
        assert low.scratch_floats >= off_best
    # more items than CTAs (twenty heads x eight sequences): no exchange, the barriers stay
    from vesta_gpu_b200.shapes import HEADS20
    low = lower_for(HEADS20, 8, 64)
    assert not low.dims['qkv_exchange'] and not low.dims['fuse_exchange']
    # switched off by hand: the reference structure of one barrier per phase
    low = lower_for(GPT2_SMALL, 8, 384, tune=dict(fuse_proj=False, qkv_exchange=False))
    assert low.barriers_per_launch == 1 + 4 * 12 and not low.dims['part_exchange']
