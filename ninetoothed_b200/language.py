"""``ninetoothed_b200.language``: the vocabulary applications are written in.

In the reference, ``ninetoothed.language.X`` is rewritten to ``triton.language.X``
in generated source (``src/ninetoothed/language.py:1-26``,
``src/ninetoothed/generation.py:849-855``).  Here an application is never
executed: the front door reads its syntax tree to decide which hand-written
kernel it denotes.  The names exist so that ``import ... as ntl`` and attribute
references resolve; calling one outside a kernel is an error.
"""

_NAMES = (
    "zeros", "full", "dot", "trans", "where", "maximum", "minimum", "max", "min", "sum", "exp", "exp2", "log",
    "log2", "sqrt", "rsqrt", "abs", "sigmoid", "cast", "arange", "rand",
)

float16 = "fp16"
bfloat16 = "bf16"
float32 = "fp32"
float64 = "fp64"
int8, int16, int32, int64 = "i8", "i16", "i32", "i64"
uint8, uint16, uint32, uint64 = "u8", "u16", "u32", "u64"


def _outside_kernel(name):
    def function(*args, **kwargs):
        raise RuntimeError(
            f"ninetoothed_b200.language.{name} describes kernel code; applications are recognised from their "
            "source, not executed"
        )

    function.__name__ = name
    return function


for _name in _NAMES:
    globals()[_name] = _outside_kernel(_name)
del _name
