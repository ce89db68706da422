"""A numpy stand-in for the slice of the jax API the reference's forward and backward paths touch.

Purpose: the golden fixtures in this folder must come from the reference's own
source, but jax is not installed where they are generated.  Installing this
stand-in into ``sys.modules`` lets ``tpa/tpa.py``, ``tpa/mha.py``,
``tpa/ring_tpa.py`` and ``tpa/tpa_test.py::reference`` be imported and executed
unmodified: every arithmetic statement they contain then runs as the same
numpy call (``jax.numpy`` is numpy), Pallas programs run one after another on
array views (what ``interpret=True`` does), ``vmap``/``scan``/``fori_loop``
are Python loops, and ``shard_map`` + ``ppermute`` run one thread per shard
with a barrier-synchronised exchange.

This is generator-side test tooling.  Nothing in the library or in the tests
that run on a GPU imports it.
"""

from __future__ import annotations

import sys
import threading
import types

import numpy as np

_tls = threading.local()


# ------------------------------------------------------------------ jax core


class _CustomVjp:
    def __init__(self, fn, nondiff_argnums=()):
        self.fn = fn
        self.__wrapped__ = fn
        self.__doc__ = fn.__doc__

    def defvjp(self, fwd, bwd):
        self.fwd, self.bwd = fwd, bwd

    def __call__(self, *a, **kw):
        return self.fn(*a, **kw)


def custom_vjp(fn=None, nondiff_argnums=()):
    if fn is None:
        return lambda f: _CustomVjp(f, nondiff_argnums)
    return _CustomVjp(fn, nondiff_argnums)


def _tree_map(f, tree):
    if isinstance(tree, (list, tuple)):
        return type(tree)(_tree_map(f, t) for t in tree)
    if tree is None:
        return None
    return f(tree)


def vmap(fn, in_axes=0, out_axes=0):
    def wrapped(*args, **kwargs):
        axes = in_axes if isinstance(in_axes, (list, tuple)) else [in_axes] * len(args)
        n = next(a.shape[ax] for a, ax in zip(args, axes) if ax is not None)
        outs = []
        for i in range(n):
            sl = [np.take(a, i, axis=ax) if ax is not None else a for a, ax in zip(args, axes)]
            kw = {key: val[i] for key, val in kwargs.items()}  # keyword operands map over axis 0
            outs.append(fn(*sl, **kw))
        first = outs[0]
        if isinstance(first, (list, tuple)):
            return type(first)(np.stack([o[j] for o in outs], axis=out_axes) for j in range(len(first)))
        return np.stack(outs, axis=out_axes)

    return wrapped


def jit(fn, **_):
    return fn


class ShapeDtypeStruct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype


# ------------------------------------------------------------------ jax.lax


def fori_loop(lo, hi, body, init):
    val = init
    for i in range(int(lo), int(hi)):
        val = body(i, val)
    return val


def scan(f, init, xs=None, length=None):
    carry = init
    ys = []
    n = len(xs) if xs is not None else length
    for i in range(n):
        carry, y = f(carry, None if xs is None else xs[i])
        ys.append(y)
    if ys and ys[0] is not None:
        return carry, np.stack(ys)
    return carry, None


def div(a, b):
    return int(a) // int(b)


class _Mesh:
    """One barrier + mailbox shared by the threads that play the shards."""

    def __init__(self, n):
        self.n = n
        self.barrier = threading.Barrier(n)
        self.box = [None] * n


def psum(x, axis_name):
    assert x == 1  # only used to read the axis size (tpa/ring_tpa.py:66)
    return _tls.mesh.n


def ppermute(x, axis_name, perm):
    mesh, me = _tls.mesh, _tls.rank
    dst = dict(perm)[me]
    mesh.barrier.wait()
    mesh.box[dst] = _tree_map(np.copy, x)
    mesh.barrier.wait()
    got = mesh.box[me]
    mesh.barrier.wait()
    return got


def run_sharded(fn, n, args, shard_axis=1):
    """shard_map over one axis: thread r runs fn on the r-th contiguous slice."""
    mesh = _Mesh(n)
    outs = [None] * n
    errs = []

    def work(r):
        _tls.mesh, _tls.rank = mesh, r
        try:
            sl = []
            for a in args:
                per = a.shape[shard_axis] // n
                idx = [slice(None)] * a.ndim
                idx[shard_axis] = slice(r * per, (r + 1) * per)
                sl.append(a[tuple(idx)])
            outs[r] = fn(*sl)
        except BaseException as e:  # noqa: BLE001 - surface it in the caller
            errs.append(e)
            mesh.barrier.abort()

    ts = [threading.Thread(target=work, args=(r,)) for r in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    if errs:
        raise errs[0]
    return np.concatenate(outs, axis=shard_axis)


# ------------------------------------------------------------------ jax.nn


def softmax(x, axis=-1):
    with np.errstate(invalid="ignore"):
        m = np.max(x, axis=axis, keepdims=True)
        e = np.exp(x - m)
        return e / np.sum(e, axis=axis, keepdims=True)


# ------------------------------------------------------------------ pallas


def program_id(axis):
    return _tls.pid[axis]


def dslice(start, size):
    return slice(int(start), int(start) + int(size))


def cdiv(a, b):
    return -(-int(a) // int(b))


class BlockSpec:
    def __init__(self, block_shape, index_map):
        self.block_shape, self.index_map = block_shape, index_map


def _block_view(arr, spec, pid):
    idx = spec.index_map(*pid)
    if not isinstance(idx, tuple):
        idx = (idx,)
    sl = tuple(slice(int(i) * s, (int(i) + 1) * s) for i, s in zip(idx, spec.block_shape))
    return arr[sl]


def atomic_add(ref, idx, val):
    # programs run one after another here, so a plain read-modify-write is the atomic add
    ref[idx] += val


def pallas_call(kernel, grid, in_specs, out_specs, out_shape, input_output_aliases=None, **_):
    single = not isinstance(out_shape, (list, tuple))
    if single:
        out_shape, out_specs = [out_shape], [out_specs]

    def run(*args):
        outs = [np.zeros(s.shape, dtype=s.dtype) for s in out_shape]
        # an aliased output starts as its input operand; operand numbers count the
        # non-None operands only (the reference numbers them that way, tpa/tpa.py:943-946)
        present = [a for a in args if a is not None]
        for src, dst in (input_output_aliases or {}).items():
            outs[dst][...] = present[src]
        for g0 in range(grid[0]):
            for g1 in range(grid[1] if len(grid) > 1 else 1):
                pid = (g0, g1)[: len(grid)]
                _tls.pid = pid
                ins = [
                    None if (a is None or sp is None) else _block_view(a, sp, pid)
                    for a, sp in zip(args, in_specs)
                ]
                os_ = [_block_view(o, sp, pid) for o, sp in zip(outs, out_specs)]
                with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
                    kernel(*ins, *os_)
        return outs[0] if single else outs

    return run


# ------------------------------------------------------------------ install


def install():
    """Put the stand-in modules into sys.modules (no-op if a real jax is importable)."""
    try:
        import jax  # noqa: F401

        if not getattr(jax, "_is_numpy_standin", False):
            raise RuntimeError("a real jax is installed; run the reference on it instead")
        return
    except ModuleNotFoundError:
        pass

    def mod(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    lax = mod("jax.lax", fori_loop=fori_loop, scan=scan, div=div, psum=psum, ppermute=ppermute)
    nn = mod("jax.nn", softmax=softmax)
    pallas = mod(
        "jax.experimental.pallas",
        program_id=program_id,
        dslice=dslice,
        cdiv=cdiv,
        BlockSpec=BlockSpec,
        pallas_call=pallas_call,
        atomic_add=atomic_add,
    )
    smap = mod("jax.experimental.shard_map", shard_map=None)
    exp = mod("jax.experimental", pallas=pallas, shard_map=smap)
    tree = mod("jax.tree", map=_tree_map)
    mod("jax.tree_util")  # jaxtyping's PyTree annotation imports it; never called here
    sharding = mod("jax.sharding", Mesh=object, PartitionSpec=tuple)
    config = types.SimpleNamespace(update=lambda *a, **k: None)
    sys.modules["jax.numpy"] = np
    mod(
        "jax",
        __path__=[],
        _is_numpy_standin=True,
        numpy=np,
        lax=lax,
        nn=nn,
        experimental=exp,
        tree=tree,
        sharding=sharding,
        config=config,
        custom_vjp=custom_vjp,
        vmap=vmap,
        jit=jit,
        ShapeDtypeStruct=ShapeDtypeStruct,
        Array=np.ndarray,
    )
