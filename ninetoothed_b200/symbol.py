"""Symbols: named compile-time quantities used inside arrangements.

Same constructor surface as the reference's ``Symbol`` and ``block_size``
(``src/ninetoothed/symbol.py:9-89, 253-265`` in the reference project): a name
plus ``constexpr`` / ``meta`` flags and optional bounds.  Here a symbol is a tiny
expression tree that can be evaluated once every name has a value; the front
door evaluates arrangements on concrete probe shapes instead of emitting code.
"""

from __future__ import annotations

import numbers
import operator

_BINARY = {
    "+": operator.add,
    "-": operator.sub,
    "*": operator.mul,
    "//": operator.floordiv,
    "%": operator.mod,
}


class Symbol:
    """A named quantity (``Symbol("BLOCK_SIZE", constexpr=True)``) or an expression of them.

    :param expr: the name (or a number, or another symbol).
    :param constexpr: the value is supplied per call, by keyword.
    :param meta: the value is a tuning meta-parameter (a block size); never a call argument.
    :param lower_bound: smallest value the symbol may take.
    :param upper_bound: largest value the symbol may take.
    :param power_of_two: whether the value must be a power of two.
    """

    def __init__(self, expr, constexpr=None, meta=None, lower_bound=None, upper_bound=None, power_of_two=None):
        if isinstance(expr, Symbol):
            self.__dict__.update(expr.__dict__)
            return
        self._op = None
        self._args = ()
        self.name = None
        self.value = None
        if isinstance(expr, numbers.Number):
            if constexpr or meta:
                raise ValueError("`constexpr` and `meta` are properties of name symbols.")
            self.value = expr
        elif isinstance(expr, str):
            if not expr.isidentifier():
                raise ValueError(f"symbol names must be identifiers, got {expr!r}")
            self.name = expr
        else:
            raise TypeError(f"cannot make a symbol from {type(expr).__name__}")
        if meta and constexpr is False:
            raise ValueError("Non-constexpr meta symbol is not supported.")
        self.meta = bool(meta)
        self.constexpr = bool(constexpr) or bool(meta)
        # Defaults of the reference (src/ninetoothed/symbol.py:59-65).
        if meta:
            defaults = (2**5, 2**10, True)
        elif constexpr:
            defaults = (1, 2**20, False)
        else:
            defaults = (None, None, None)
        self.lower_bound = lower_bound if lower_bound is not None else defaults[0]
        self.upper_bound = upper_bound if upper_bound is not None else defaults[1]
        self.power_of_two = power_of_two if power_of_two is not None else defaults[2]

    @classmethod
    def _expression(cls, op, *args):
        node = cls.__new__(cls)
        node._op, node._args = op, tuple(a if isinstance(a, Symbol) else Symbol(a) for a in args)
        node.name = node.value = None
        node.meta = node.constexpr = False
        node.lower_bound = node.upper_bound = node.power_of_two = None
        return node

    # -- evaluation -----------------------------------------------------------
    def names(self):
        """Name symbols this expression depends on."""
        if self.name is not None:
            return {self}
        found = set()
        for arg in self._args:
            found |= arg.names()
        return found

    def evaluate(self, env):
        """Value under ``env``, a mapping from symbol name to number."""
        if self.value is not None:
            return self.value
        if self.name is not None:
            if self.name not in env:
                raise KeyError(f"symbol {self.name!r} has no value")
            return env[self.name]
        left, right = (arg.evaluate(env) for arg in self._args)
        return _BINARY[self._op](left, right)

    # -- arithmetic -------------------------------------------------------------
    def __add__(self, other):
        return Symbol._expression("+", self, other)

    def __radd__(self, other):
        return Symbol._expression("+", other, self)

    def __sub__(self, other):
        return Symbol._expression("-", self, other)

    def __rsub__(self, other):
        return Symbol._expression("-", other, self)

    def __mul__(self, other):
        return Symbol._expression("*", self, other)

    def __rmul__(self, other):
        return Symbol._expression("*", other, self)

    def __floordiv__(self, other):
        return Symbol._expression("//", self, other)

    def __rfloordiv__(self, other):
        return Symbol._expression("//", other, self)

    def __mod__(self, other):
        return Symbol._expression("%", self, other)

    def __eq__(self, other):
        if isinstance(other, Symbol):
            return repr(self) == repr(other)
        if isinstance(other, numbers.Number):
            return self.value is not None and self.value == other
        return NotImplemented

    def __hash__(self):
        return hash(repr(self))

    def __repr__(self):
        if self.value is not None:
            return repr(self.value)
        if self.name is not None:
            return self.name
        return f"({self._args[0]!r} {self._op} {self._args[1]!r})"

    @staticmethod
    def is_name(obj):
        return isinstance(obj, Symbol) and obj.name is not None


def block_size(lower_bound=None, upper_bound=None):
    """A fresh block-size meta-parameter (``src/ninetoothed/symbol.py:253-265``)."""
    name = f"BLOCK_SIZE_{block_size._count}"
    block_size._count += 1
    return Symbol(name, meta=True, lower_bound=lower_bound, upper_bound=upper_bound)


block_size._count = 0
