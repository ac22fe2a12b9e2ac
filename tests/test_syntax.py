"""The front end: grammar of the reference language (GRAMMAR.md:17-43)."""
import os

import pytest

from vesta_gpu_b200 import syntax as sx, PROGRAMS
from vesta_gpu_b200.program_text import decode_program
from vesta_gpu_b200.shapes import GPT2_SMALL, GPT2_XL, TINY


def test_expression_precedence():
    e = sx.parse_expression('a + b * c - d / 2')
    assert e == sx.Bin('-', sx.Bin('+', sx.Name('a'), sx.Bin('*', sx.Name('b'), sx.Name('c'))),
                       sx.Bin('/', sx.Name('d'), sx.Num(2)))
    assert sx.parse_expression('-x * y') == sx.Bin('*', sx.Neg(sx.Name('x')), sx.Name('y'))
    assert sx.parse_expression('a == b + 1') == sx.Bin('==', sx.Name('a'), sx.Bin('+', sx.Name('b'), sx.Num(1)))


def test_numbers():
    assert sx.parse_expression('0.00001') == sx.Num(1e-5)
    assert sx.parse_expression('3') == sx.Num(3) and isinstance(sx.parse_expression('3').value, int)
    assert sx.parse_expression('2e-3') == sx.Num(2e-3)
    assert sx.parse_expression('1.5e2') == sx.Num(150.0)


def test_fold_fork_index_call():
    e = sx.parse_expression('fold min n: fork logit[n] == best ? n : 50257')
    assert e == sx.Fold('min', 'n', sx.Fork(sx.Bin('==', sx.Index('logit', (sx.Name('n'),)), sx.Name('best')),
                                            sx.Name('n'), sx.Num(50257)))
    e = sx.parse_expression('(fold sum d: a[d] * w[l, d, j]) + b[l, j]')
    assert isinstance(e, sx.Bin) and isinstance(e.lhs, sx.Fold) and e.lhs.axis == 'd'
    assert sx.parse_expression('exp(x - m)') == sx.Call('exp', sx.Bin('-', sx.Name('x'), sx.Name('m')))
    assert sx.parse_expression('q[h * 64 + e]') == sx.Index('q', (sx.Bin('+', sx.Bin('*', sx.Name('h'), sx.Num(64)), sx.Name('e')),))
    # a name that is also a function is a plain name when not called
    assert sx.parse_expression('exp + 1') == sx.Bin('+', sx.Name('exp'), sx.Num(1))


def test_statements():
    prog = sx.parse('''
        residue x            # scalar
        axis d = 4
        axis s = t + 1
        residue w[s, d]
        residue k[l, t, h] <- q[8 + h]
        y[d] = w[x, d]
        r[d] = fold step l: y as z
            u[d] = z[d] * 2
            -> u
        end
    ''')
    assert prog[0] == sx.Receive('x', ())
    assert prog[1] == sx.AxisDef('d', sx.Num(4))
    assert prog[2] == sx.AxisDef('s', sx.Bin('+', sx.Name('t'), sx.Num(1)))
    assert prog[3] == sx.Receive('w', ('s', 'd'))
    assert isinstance(prog[4], sx.Emit) and prog[4].name == 'k' and len(prog[4].at) == 3
    step = prog[6]
    assert isinstance(step, sx.StepFold) and step.axis == 'l' and step.carry == 'z' and step.init == sx.Name('y')
    assert step.result == sx.Name('u') and len(step.body) == 1


@pytest.mark.parametrize('bad', ['a = = 1', 'a = b +', 'a[ = 1', 'a = (b', 'a = b ? c', 'a = 1 $ 2', 'end', '-> x',
                                 'r = fold step l: y as z\n  u = z\nend', 'r = fold step l: y as z\n -> z'])
def test_syntax_errors(bad):
    with pytest.raises(SyntaxError):
        sx.parse(bad)


def test_shipped_programs_match_generator():
    assert (PROGRAMS / 'gpt2.vst').read_text() == decode_program(GPT2_SMALL)
    assert (PROGRAMS / 'gpt2_xl.vst').read_text() == decode_program(GPT2_XL)
    for sh in (GPT2_SMALL, GPT2_XL, TINY):
        prog = sx.parse(decode_program(sh))
        assert sum(isinstance(s, sx.StepFold) for s in prog) == 1


# a checkout of the reference (VESTA_REFERENCE) or the copy oracle/make_ref.py installs
REF_PROGRAM = next((p for p in (os.path.join(os.environ.get('VESTA_REFERENCE', ''), 'vesta', 'programs', 'gpt2.vst'),
                                os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'oracle', '_ref', 'vesta', 'programs', 'gpt2.vst'))
                    if os.path.exists(p)), '')


@pytest.mark.skipif(not os.path.exists(REF_PROGRAM), reason='reference checkout not present')
def test_same_tree_as_reference_program():
    """the program the reference ships and the generated text are the same statements"""
    ref = open(REF_PROGRAM, encoding='utf-8').read()
    assert sx.parse(ref) == sx.parse(decode_program(GPT2_SMALL))


def test_drop_in_package_offers_interp():
    """vesta.interp of the drop-in package: `parse` is this backend's front end; `run` is the reference's CPU
    interpreter when a copy of the reference is installed, and says so when it is not"""
    import numpy as np
    import vesta.interp as vi
    assert vi.parse is sx.parse
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if os.path.exists(os.path.join(here, 'oracle', '_ref', 'vesta', 'interp.py')):
        env = vi.run('residue a\naxis i = 3\nb[i] = a[i] + a[i]\n', {'a': np.arange(3, dtype=np.float32)})
        assert np.array_equal(np.asarray(env['b'][0]), [0, 2, 4])
    else:
        with pytest.raises(ImportError):
            vi.run('', {})
