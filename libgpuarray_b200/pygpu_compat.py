"""pygpu's reduction front end on top of GpuReduction_*.

The reference implements ndgpuarray.sum/prod/all/any in Python: `reduce1`
(pygpu/reduction.py:294-319) renders a mako template into a `reduk` kernel.
This module provides the same two callables, `reduce1` and
`ReductionKernel(context, dtype_out, neutral, reduce_expr, redux, map_expr,
arguments)`, but runs them through the library's C engines: GpuReduction_* for
one array with a plain operator, GpuMapReduction_* for a map expression over
several (broadcastable) arguments. `install()` puts them in place of pygpu's own, which lifts
the template's limits (32-bit sizes, no float16, one block for full
reductions) and removes the mako dependency:

    import pygpu
    from libgpuarray_b200 import pygpu_compat
    pygpu_compat.install()
    x.sum(axis=1)        # ndgpuarray method -> GpuReduction_call
    x.argmax(axis=1)     # added: max / min / argmax / argmin (pygpu has them commented out)

pygpu arrays are handed over without copies: `GpuContext.ptr` is the
gpucontext*, `GpuArray.gpudata` the device address of element [0,...,0].
"""
import re

import numpy as np

from . import api

_OPS = {"+": api.GA_REDUCE_SUM, "*": api.GA_REDUCE_PROD, "&&": api.GA_REDUCE_ALL,
        "||": api.GA_REDUCE_ANY, "&": api.GA_REDUCE_AND, "|": api.GA_REDUCE_OR,
        "^": api.GA_REDUCE_XOR}
_EXPRS = {"a+b": api.GA_REDUCE_SUM, "a*b": api.GA_REDUCE_PROD, "a&&b": api.GA_REDUCE_ALL,
          "a||b": api.GA_REDUCE_ANY, "max(a,b)": api.GA_REDUCE_MAX, "min(a,b)": api.GA_REDUCE_MIN,
          "a&b": api.GA_REDUCE_AND, "a|b": api.GA_REDUCE_OR, "a^b": api.GA_REDUCE_XOR}
_contexts = {}
_operators = {}


def _ctx(pygpu_context):
    key = int(pygpu_context.ptr)
    if key not in _contexts:
        _contexts[key] = api.Context.borrow(key)
    return _contexts[key]


def _wrap(ctx, a):
    return api.GpuArray.from_pointer(ctx, int(a.gpudata), a.shape, a.dtype, strides=a.strides)


def _run(opcode, ary, redux, out_type, out):
    import pygpu
    out_type = np.dtype(out_type)
    axes = [i for i, r in enumerate(redux) if r]
    if not axes:
        raise ValueError("Reduction is along no axes")
    kept = tuple(d for d, r in zip(ary.shape, redux) if not r)
    if out is None:
        out = pygpu.gpuarray.empty(kept, dtype=out_type, context=ary.context, cls=type(ary))
    else:
        if out.shape != kept or out.dtype != out_type:
            raise TypeError("Out array is not of expected type (expected %s %s, got %s %s)" %
                            (kept, out_type, out.shape, out.dtype))
    ctx = _ctx(ary.context)
    key = (int(ary.context.ptr), opcode, ary.dtype.str)
    if key not in _operators:
        _operators[key] = api.GpuReduction(ctx, opcode, ary.dtype)
    if ary.size == 0 and opcode in (api.GA_REDUCE_MAX, api.GA_REDUCE_MIN):
        raise ValueError("min/max of an empty array")
    _operators[key](_wrap(ctx, out), None, _wrap(ctx, ary), axes)
    return out


def _axis_mask(nd, axis):
    if axis is None:
        return [True] * nd
    redux = [False] * nd
    if not isinstance(axis, (list, tuple)):
        axis = (axis,)
    for ax in axis:
        if ax < 0:
            ax += nd
        if ax < 0 or ax >= nd:
            raise ValueError("axis out of bounds")
        redux[ax] = True
    return redux


def _minmax(ary, opcode, axis, want_value, want_index):
    """max / min / argmax / argmin, which pygpu leaves commented out
    (pygpu/_array.py:264-280). A tuple of axes is reduced as in
    GpuArray_maxandargmax: the index is the flattened position over the listed
    axes, in the order listed."""
    import pygpu
    if ary.size == 0:
        raise ValueError("min/max of an empty array")
    if ary.ndim == 0:
        ary = ary.reshape((1,))
    axes = list(range(ary.ndim)) if axis is None else \
        [a + ary.ndim if a < 0 else a for a in (axis if isinstance(axis, (list, tuple)) else (axis,))]
    kept = tuple(d for i, d in enumerate(ary.shape) if i not in axes)
    ctx = _ctx(ary.context)
    key = (int(ary.context.ptr), opcode, ary.dtype.str)
    if key not in _operators:
        _operators[key] = api.GpuReduction(ctx, opcode, ary.dtype)
    val = idx = None
    if want_value:
        val = pygpu.gpuarray.empty(kept, dtype=ary.dtype, context=ary.context, cls=type(ary))
    if want_index:
        idx = pygpu.gpuarray.empty(kept, dtype="int64", context=ary.context, cls=type(ary))
    _operators[key](_wrap(ctx, val) if want_value else None, _wrap(ctx, idx) if want_index else None,
                    _wrap(ctx, ary), axes)
    return val, idx


def amax(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_MAX, axis, True, False)[0]


def amin(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_MIN, axis, True, False)[0]


def argmax(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_ARGMAX, axis, False, True)[1]


def argmin(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_ARGMIN, axis, False, True)[1]


def maxandargmax(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_MAXANDARGMAX, axis, True, True)


def minandargmin(ary, axis=None):
    return _minmax(ary, api.GA_REDUCE_MINANDARGMIN, axis, True, True)


def reduce1(ary, op, neutral, out_type, axis=None, out=None, oper=None):
    """Same signature and axis handling as pygpu.reduction.reduce1."""
    nd = ary.ndim
    if axis is None:
        redux = [True] * nd
    else:
        redux = [False] * nd
        if not isinstance(axis, (list, tuple)):
            axis = (axis,)
        for ax in axis:
            if ax < 0:
                ax += nd
            if ax < 0 or ax >= nd:
                raise ValueError("axis out of bounds")
            redux[ax] = True
    opcode = _EXPRS.get(oper.replace(" ", "")) if oper is not None else _OPS.get(op)
    if opcode is None:
        raise NotImplementedError("reduction operator %r" % (oper or op))
    return _run(opcode, ary, redux, out_type, out)


_INDEX_RE = re.compile(r"([a-zA-Z_][a-zA-Z0-9_]*)\[i\]")


def _parse_c_arguments(text):
    """'float *a, double *b, int n' -> [(name, dtype, is_array)], the C argument
    list form that pygpu.reduction.ReductionKernel also accepts."""
    names = {"float": np.float32, "double": np.float64, "int": np.int32, "unsigned int": np.uint32,
             "long": np.int64, "unsigned long": np.uint64, "short": np.int16,
             "unsigned short": np.uint16, "char": np.int8, "unsigned char": np.uint8,
             "bool": np.bool_, "ga_float": np.float32, "ga_double": np.float64, "ga_int": np.int32,
             "ga_uint": np.uint32, "ga_long": np.int64, "ga_ulong": np.uint64,
             "ga_short": np.int16, "ga_ushort": np.uint16, "ga_byte": np.int8,
             "ga_ubyte": np.uint8, "ga_bool": np.bool_, "ga_half": np.float16}
    out = []
    for piece in text.split(","):
        piece = piece.replace("const", " ").replace("GLOBAL_MEM", " ").strip()
        is_array = "*" in piece
        piece = piece.replace("*", " ")
        words = piece.split()
        if len(words) < 2 or " ".join(words[:-1]) not in names:
            raise ValueError("cannot parse C argument %r" % piece)
        out.append((words[-1], np.dtype(names[" ".join(words[:-1])]), is_array))
    return out


class ReductionKernel(object):
    """pygpu.reduction.ReductionKernel (pygpu/reduction.py:137-291) on the
    library's engines: one array with a plain operator goes to
    GpuReduction_call; a map expression and / or several (broadcastable)
    arguments go to GpuMapReduction_call, where map and reduction are one pass
    over memory."""

    def __init__(self, context, dtype_out, neutral, reduce_expr, redux, map_expr=None,
                 arguments=None, preamble="", init_nd=None):
        if not any(redux):
            raise ValueError("Reduction is along no axes")
        self.context = context
        self.redux = list(redux)
        self.dtype_out = np.dtype(dtype_out)
        self.opcode = None
        self.mapred = None
        if isinstance(arguments, str):
            arguments = _parse_c_arguments(arguments)
        elif arguments is not None:
            arguments = [(a.name, np.dtype(a.dtype), bool(a.isarray())) for a in arguments]
        plain = map_expr is None or (arguments is None and map_expr.replace(" ", "") == "a[i]") or \
            (arguments is not None and len(arguments) == 1 and
             map_expr.replace(" ", "") == "%s[i]" % arguments[0][0])
        if plain and (arguments is None or len(arguments) == 1):
            self.opcode = _EXPRS.get(reduce_expr.replace(" ", ""))
        if self.opcode is not None:
            return
        if arguments is None:
            arguments = [("_reduce_input", self.dtype_out, True)]
        if map_expr is None:
            if len(arguments) != 1:
                raise ValueError("Don't know what to do with more than one argument. Specify "
                                 "map_expr to explicitly state what you want.")
            map_expr = "%s[i]" % arguments[0][0]
        if not any(isarr for _, _, isarr in arguments):
            raise ValueError("ReductionKernel can only be used with functions that have at least "
                             "one vector argument.")
        self.arguments = arguments
        spec = [(name, dt, api.GE_READ if isarr else api.GE_SCALAR) for name, dt, isarr in arguments]
        f16 = self.dtype_out == np.float16 or any(dt == np.float16 for _, dt, _ in arguments)
        self.mapred = api.GpuMapReduction(_ctx(context), _INDEX_RE.sub(r"\g<1>", map_expr), reduce_expr,
                                          neutral, self.dtype_out, spec, preamble=preamble or "",
                                          convert_f16=f16)

    def __call__(self, *args, **kwargs):
        import pygpu
        broadcast = kwargs.pop("broadcast", None)
        out = kwargs.pop("out", None)
        if kwargs:
            raise TypeError("Unexpected keyword argument: %s" % list(kwargs)[0])
        if self.mapred is None:
            (ary,) = args
            if len(self.redux) != ary.ndim:
                raise ValueError("redux mask does not match the array rank")
            return _run(self.opcode, ary, self.redux, self.dtype_out, out)
        if len(args) != len(self.arguments):
            raise TypeError("expected %d arguments" % len(self.arguments))
        arrays = [a for a, (_, _, isarr) in zip(args, self.arguments) if isarr]
        nd = max(a.ndim for a in arrays)
        if len(self.redux) != nd:
            raise ValueError("redux mask does not match the rank of the arguments")
        shape = [1] * nd
        for a in arrays:
            if a.ndim != nd:
                raise ValueError("arguments differ in rank")
            for j, d in enumerate(a.shape):
                if d != 1:
                    if shape[j] not in (1, d):
                        raise ValueError("shapes cannot be combined")
                    shape[j] = d
        kept = tuple(d for d, r in zip(shape, self.redux) if not r)
        if out is None:
            out = pygpu.gpuarray.empty(kept, dtype=self.dtype_out, context=self.context,
                                       cls=type(arrays[0]))
        elif out.shape != kept or out.dtype != self.dtype_out:
            raise TypeError("Out array is not of expected type (expected %s %s, got %s %s)" %
                            (kept, self.dtype_out, out.shape, out.dtype))
        ctx = _ctx(self.context)
        wrapped = [_wrap(ctx, a) if isarr else a for a, (_, _, isarr) in zip(args, self.arguments)]
        axes = [i for i, r in enumerate(self.redux) if r]
        try:
            self.mapred(_wrap(ctx, out), *wrapped, axes=axes, broadcast=bool(broadcast),
                        padshape=False)
        except api.GpuArrayException as e:
            if e.code == api.GA_VALUE_ERROR:
                raise ValueError(str(e))
            raise
        return out


def install():
    """Replaces pygpu's template-based reduction entry points by these."""
    import pygpu.reduction
    import pygpu._array
    pygpu.reduction.reduce1 = reduce1
    pygpu.reduction.ReductionKernel = ReductionKernel
    pygpu._array.reduce1 = reduce1
    for name, fn in (("max", amax), ("min", amin), ("argmax", argmax), ("argmin", argmin)):
        setattr(pygpu._array.ndgpuarray, name, fn)
