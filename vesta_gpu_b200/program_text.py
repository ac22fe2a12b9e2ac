"""Text of the decode-step program for any model shape.

The reference ships one program with GPT-2 small's sizes written into it
(vesta/programs/gpt2.vst:6-12,39-40,48-49). The statements are the same for every width and
depth of the family, so the text is generated from a Shape; `programs/gpt2.vst` and
`programs/gpt2_xl.vst` are the output of this module for the two benchmark shapes.
"""
from .shapes import Shape, GPT2_SMALL, GPT2_XL
from . import PROGRAMS


def _num(v):
    return repr(int(v)) if float(v) == int(v) else repr(float(v))


ADDITIVE = ('ln1b', 'qkvb', 'ob', 'ln2b', 'fcb', 'pb', 'lnfb')     # the shifts and biases a program may leave out


def decode_program(sh: Shape, eps=0.00001, without=()) -> str:
    """without: names from ADDITIVE; the program then neither receives nor adds those parameters (a model without
    biases, a LayerNorm without shift)"""
    D, H, E, F, N, J, L = sh.D, sh.H, sh.E, sh.F, sh.N, sh.J, sh.L
    text = _decode_program(sh, eps)
    if not without:
        return text
    terms = {'ln1b': ' + ln1b[l, d]', 'qkvb': ' + qkvb[l, j]', 'ob': ' + ob[l, d]', 'ln2b': ' + ln2b[l, d]',
             'fcb': ' + fcb[l, f]', 'pb': ' + pb[l, d]', 'lnfb': ' + lnfb[d]'}
    out = []
    for line in text.split('\n'):
        for name in without:
            if line.startswith(f'residue {name}['):
                line = None
                break
            if line.endswith(terms[name]):
                line = line[:-len(terms[name])]
        if line is not None:
            out.append(line)
    return '\n'.join(out)


def _decode_program(sh: Shape, eps=0.00001) -> str:
    D, H, E, F, N, J, L = sh.D, sh.H, sh.E, sh.F, sh.N, sh.J, sh.L
    scale = _num(E ** 0.5)
    lines = [
        f'# {sh.name}: one decode step ({L} layers, width {D}, {H} heads of {E}, MLP {F}, vocabulary {N})',
        'residue x',
        'residue t',
        f'axis d = {D}', f'axis h = {H}', f'axis e = {E}', f'axis f = {F}', f'axis n = {N}',
        f'axis j = {J}', f'axis l = {L}', 'axis s = t + 1',
        'residue wte[n, d]', 'residue wpe[s, d]',
        'residue ln1w[l, d]', 'residue ln1b[l, d]', 'residue qkvw[l, d, j]', 'residue qkvb[l, j]',
        'residue ow[l, d, d]', 'residue ob[l, d]', 'residue ln2w[l, d]', 'residue ln2b[l, d]',
        'residue fcw[l, d, f]', 'residue fcb[l, f]', 'residue pw[l, f, d]', 'residue pb[l, d]',
        'residue lnfw[d]', 'residue lnfb[d]',
        'residue keys[l, s, h, e]', 'residue vals[l, s, h, e]',
        '',
        'z0[d] = wte[x, d] + wpe[t, d]',
        'zL[d] = fold step l: z0 as z',
        f'    m1 = fold sum d: z[d] / {D}',
        f'    v1 = fold sum d: (z[d] - m1) * (z[d] - m1) / {D}',
        f'    a[d] = (z[d] - m1) / sqrt(v1 + {eps:.5f}) * ln1w[l, d] + ln1b[l, d]',
        '    qkv[j] = (fold sum d: a[d] * qkvw[l, d, j]) + qkvb[l, j]',
        f'    q[h, e] = qkv[h * {E} + e]',
        f'    residue keys[l, t, h, e] <- qkv[{D} + h * {E} + e]',
        f'    residue vals[l, t, h, e] <- qkv[{2 * D} + h * {E} + e]',
        f'    sc[h, s] = (fold sum e: q[h, e] * keys[l, s, h, e]) / {scale}',
        '    mx[h] = fold max s: sc[h, s]',
        '    ex[h, s] = exp(sc[h, s] - mx[h])',
        '    w[h, s] = ex[h, s] / (fold sum s: ex[h, s])',
        '    o[h, e] = fold sum s: w[h, s] * vals[l, s, h, e]',
        f'    oo[d] = fold sum h: (fold sum e: o[h, e] * ow[l, h * {E} + e, d])',
        '    z1[d] = z[d] + oo[d] + ob[l, d]',
        f'    m2 = fold sum d: z1[d] / {D}',
        f'    v2 = fold sum d: (z1[d] - m2) * (z1[d] - m2) / {D}',
        f'    b[d] = (z1[d] - m2) / sqrt(v2 + {eps:.5f}) * ln2w[l, d] + ln2b[l, d]',
        '    u[f] = (fold sum d: b[d] * fcw[l, d, f]) + fcb[l, f]',
        '    g[f] = 0.5 * u[f] * (1 + tanh(0.7978845608028654 * (u[f] + 0.044715 * u[f] * u[f] * u[f])))',
        '    z2[d] = z1[d] + (fold sum f: g[f] * pw[l, f, d]) + pb[l, d]',
        '    -> z2',
        'end',
        f'm3 = fold sum d: zL[d] / {D}',
        f'v3 = fold sum d: (zL[d] - m3) * (zL[d] - m3) / {D}',
        f'c[d] = (zL[d] - m3) / sqrt(v3 + {eps:.5f}) * lnfw[d] + lnfb[d]',
        'logit[n] = fold sum d: c[d] * wte[n, d]',
        'best = fold max n: logit[n]',
        f'next = fold min n: fork logit[n] == best ? n : {N}',
    ]
    return '\n'.join(lines) + '\n'


def write_programs():
    for sh, fn in ((GPT2_SMALL, 'gpt2.vst'), (GPT2_XL, 'gpt2_xl.vst')):
        (PROGRAMS / fn).write_text(decode_program(sh), encoding='utf-8')


if __name__ == '__main__':
    write_programs()
