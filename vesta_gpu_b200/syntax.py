"""Front end of the four-form language: text -> statement tree.

Accepts the grammar of the reference (GRAMMAR.md:17-43, parsed there by vesta/interp.py:16-129):
line-oriented statements (`axis`, `residue` receive / emit, named values, `fold step ... end`
blocks closed by `-> e`), and expressions with fork, fold sum|max|min, one comparison level,
+ - * /, unary minus, indexing and the functions exp / tanh / sqrt.

The tree is made of small frozen dataclasses so that it can be compared structurally; the
placement pass (lower.py) recognises a program by matching these trees against statement
patterns, in which a name that starts with `$` is a wildcard.
"""
from dataclasses import dataclass
from typing import Tuple, Union

FOLD_OPS = ('sum', 'max', 'min')
FUNCS = ('exp', 'tanh', 'sqrt')
COMPARE = ('==', '<=', '>=', '<', '>')


# ------------------------------------------------------------------ tree
@dataclass(frozen=True)
class Num:
    value: Union[int, float]


@dataclass(frozen=True)
class Name:
    id: str


@dataclass(frozen=True)
class Neg:
    arg: object


@dataclass(frozen=True)
class Call:
    fn: str
    arg: object


@dataclass(frozen=True)
class Bin:
    op: str
    lhs: object
    rhs: object


@dataclass(frozen=True)
class Index:
    base: str
    at: Tuple[object, ...]


@dataclass(frozen=True)
class Fold:
    op: str
    axis: str
    body: object


@dataclass(frozen=True)
class Fork:
    cond: object
    then: object
    other: object


@dataclass(frozen=True)
class AxisDef:
    name: str
    extent: object


@dataclass(frozen=True)
class Receive:
    name: str
    axes: Tuple[str, ...]


@dataclass(frozen=True)
class Emit:
    name: str
    at: Tuple[object, ...]
    value: object


@dataclass(frozen=True)
class Let:
    name: str
    axes: Tuple[str, ...]
    value: object


@dataclass(frozen=True)
class StepFold:
    name: str
    axes: Tuple[str, ...]
    axis: str                 # the axis stepped over
    init: object
    carry: str
    body: Tuple[object, ...]  # statements
    result: object            # the expression after `->`


# ------------------------------------------------------------------ scanner
def scan(line, wild=False):
    """one source line -> list of (kind, value); kinds: num, id, op"""
    out, i, n = [], 0, len(line)
    two = ('<-', '->', '==', '<=', '>=')
    while i < n:
        ch = line[i]
        if ch in ' \t':
            i += 1
            continue
        if ch == '#':
            break
        if ch.isdigit():
            k = i
            while k < n and line[k].isdigit():
                k += 1
            is_float = False
            if k < n and line[k] == '.':
                is_float = True
                k += 1
                while k < n and line[k].isdigit():
                    k += 1
            if k < n and line[k] in 'eE':
                m = k + 1
                if m < n and line[m] in '+-':
                    m += 1
                if m < n and line[m].isdigit():
                    is_float = True
                    while m < n and line[m].isdigit():
                        m += 1
                    k = m
            text = line[i:k]
            out.append(('num', float(text) if is_float else int(text)))
            i = k
            continue
        if ch.isalpha() or ch == '_' or (wild and ch == '$'):
            k = i + 1
            while k < n and (line[k].isalnum() or line[k] == '_'):
                k += 1
            out.append(('id', line[i:k]))
            i = k
            continue
        if line[i:i + 2] in two:
            out.append(('op', line[i:i + 2]))
            i += 2
            continue
        if ch in '[](),:+-*/?<>=':
            out.append(('op', ch))
            i += 1
            continue
        raise SyntaxError(f'bad character {ch!r}')
    return out


class _Cursor:
    def __init__(self, toks):
        self.toks, self.pos = toks, 0

    def at(self, k=0):
        p = self.pos + k
        return self.toks[p] if p < len(self.toks) else ('end', None)

    def value(self, k=0):
        return self.at(k)[1]

    def next(self):
        tok = self.at()
        self.pos += 1
        return tok

    def expect(self, v):
        tok = self.next()
        if tok[1] != v:
            raise SyntaxError(f'expected {v!r}, found {tok[1]!r}')

    def ident(self):
        kind, v = self.next()
        if kind != 'id':
            raise SyntaxError(f'expected a name, found {v!r}')
        return v

    def end(self):
        return self.pos >= len(self.toks)

    # expression grammar, lowest binding first
    def expr(self):
        if self.at() == ('id', 'fork'):
            self.next()
            cond = self.compare()
            self.expect('?')
            then = self.expr()
            self.expect(':')
            return Fork(cond, then, self.expr())
        if self.at() == ('id', 'fold') and self.value(1) in FOLD_OPS:
            self.next()
            op = self.ident()
            axis = self.ident()
            self.expect(':')
            return Fold(op, axis, self.expr())
        return self.compare()

    def compare(self):
        lhs = self.additive()
        if self.at()[0] == 'op' and self.value() in COMPARE:
            op = self.next()[1]
            return Bin(op, lhs, self.additive())
        return lhs

    def additive(self):
        lhs = self.term()
        while self.at() in (('op', '+'), ('op', '-')):
            op = self.next()[1]
            lhs = Bin(op, lhs, self.term())
        return lhs

    def term(self):
        lhs = self.unary()
        while self.at() in (('op', '*'), ('op', '/')):
            op = self.next()[1]
            lhs = Bin(op, lhs, self.unary())
        return lhs

    def unary(self):
        if self.at() == ('op', '-'):
            self.next()
            return Neg(self.unary())
        return self.postfix()

    def postfix(self):
        node = self.primary()
        if self.at() == ('op', '['):
            if not isinstance(node, Name):
                raise SyntaxError('only a named value can be indexed')
            self.next()
            at = [self.expr()]
            while self.at() == ('op', ','):
                self.next()
                at.append(self.expr())
            self.expect(']')
            return Index(node.id, tuple(at))
        return node

    def primary(self):
        kind, v = self.next()
        if kind == 'num':
            return Num(v)
        if kind == 'op' and v == '(':
            inner = self.expr()
            self.expect(')')
            return inner
        if kind == 'id':
            if v in FUNCS and self.at() == ('op', '('):
                self.next()
                arg = self.expr()
                self.expect(')')
                return Call(v, arg)
            return Name(v)
        raise SyntaxError(f'unexpected {v!r}')

    def name_list(self):
        names = [self.ident()]
        while self.at() == ('op', ','):
            self.next()
            names.append(self.ident())
        return tuple(names)


def parse_expression(text, wild=False):
    cur = _Cursor(scan(text, wild))
    node = cur.expr()
    if not cur.end():
        raise SyntaxError(f'trailing {cur.value()!r}')
    return node


def _statement(cur, toks):
    """one non-block statement from a cursor at its first token; a `fold step` header returns
    ('open', name, axes, axis, init, carry)"""
    head = cur.at()
    if head == ('op', '->'):
        cur.next()
        node = ('result', cur.expr())
    elif head == ('id', 'axis'):
        cur.next()
        name = cur.ident()
        cur.expect('=')
        node = AxisDef(name, cur.expr())
    elif head == ('id', 'residue'):
        cur.next()
        name = cur.ident()
        if cur.end():
            return Receive(name, ())
        cur.expect('[')
        if ('op', '<-') in toks:
            at = [cur.expr()]
            while cur.at() == ('op', ','):
                cur.next()
                at.append(cur.expr())
            cur.expect(']')
            cur.expect('<-')
            node = Emit(name, tuple(at), cur.expr())
        else:
            axes = cur.name_list()
            cur.expect(']')
            node = Receive(name, axes)
    else:
        name = cur.ident()
        axes = ()
        if cur.at() == ('op', '['):
            cur.next()
            axes = cur.name_list()
            cur.expect(']')
        cur.expect('=')
        if cur.at() == ('id', 'fold') and cur.at(1) == ('id', 'step'):
            cur.next()
            cur.next()
            axis = cur.ident()
            cur.expect(':')
            # the initial value runs up to the last `as`
            last_as = max((i for i in range(cur.pos, len(toks)) if toks[i] == ('id', 'as')), default=None)
            if last_as is None:
                raise SyntaxError('fold step needs `as NAME`')
            init_cur = _Cursor(toks[cur.pos:last_as])
            init = init_cur.expr()
            if not init_cur.end():
                raise SyntaxError(f'trailing {init_cur.value()!r}')
            cur.pos = last_as + 1
            carry = cur.ident()
            node = ('open', name, axes, axis, init, carry)
        else:
            node = Let(name, axes, cur.expr())
    if not cur.end():
        raise SyntaxError(f'trailing {cur.value()!r}')
    return node


def parse(text, wild=False):
    """program text -> tuple of statements"""
    frames = [dict(body=[], header=None, result=None)]
    for lineno, raw in enumerate(text.splitlines(), 1):
        try:
            toks = scan(raw, wild)
            if not toks:
                continue
            if toks == [('id', 'end')]:
                if len(frames) == 1:
                    raise SyntaxError('`end` without a fold step')
                fr = frames.pop()
                if fr['result'] is None:
                    raise SyntaxError('fold step without `->`')
                _, name, axes, axis, init, carry = fr['header']
                frames[-1]['body'].append(StepFold(name, axes, axis, init, carry, tuple(fr['body']), fr['result']))
                continue
            node = _statement(_Cursor(toks), toks)
            if isinstance(node, tuple) and node[0] == 'open':
                frames.append(dict(body=[], header=node, result=None))
            elif isinstance(node, tuple) and node[0] == 'result':
                if len(frames) == 1 or frames[-1]['result'] is not None:
                    raise SyntaxError('`->` belongs once inside a fold step')
                frames[-1]['result'] = node[1]
            else:
                frames[-1]['body'].append(node)
        except SyntaxError as err:
            raise SyntaxError(f'line {lineno}: {raw.strip()!r}: {err}') from None
    if len(frames) != 1:
        raise SyntaxError('missing end')
    return tuple(frames[0]['body'])
