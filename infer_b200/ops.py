"""Operators of the paged KV-cache path, behind the reference's call signatures.

* ``store_kvcache(key, value, k_cache, v_cache, slot_mapping)`` - same arguments and the
  same stride asserts as the reference's Triton wrapper (infer/ops/attention.py:38-45).
* ``paged_attn_decode`` / ``paged_attn_prefill`` - the two calls the reference makes into
  the flash_attn package (infer/ops/attention.py:110-121), with the keyword names it uses.
* ``flash_attn_prefill(Q, K, V, O)`` - the reference's own dense op (src/bindings.cpp:9).

Every op launches hand-written sm_100a kernels through the C ABI on the current CUDA
stream and is also registered as ``torch.ops._C.<name>`` with out-parameter schemas in
the style of src/bindings.cpp:4-23.  Nothing here computes on the CPU or through PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib

_POOLS: dict = {}
_CHECK = os.environ.get("INFER_B200_CHECK") == "1"    # debugging: read the device status word after each call


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on_device:
    """``torch.cuda.device(dev)`` without its cost when ``dev`` is already current (the usual case)."""

    __slots__ = ("guard",)

    def __init__(self, device):
        self.guard = None if torch.cuda.current_device() == device.index else torch.cuda.device(device)

    def __enter__(self):
        if self.guard is not None:
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


# The three attention entry points are reached through these one-line functions so that the test
# suite can route a call to the library's self-test entry points (infer_b200/selftest.py).
def _call_decode(lib, *args):
    return lib.infer_paged_decode(*args)


def _call_prefill(lib, *args):
    return lib.infer_paged_prefill(*args)


def _call_dense(lib, *args):
    return lib.infer_flash_attn_prefill(*args)


class _Scratch:
    """Zero-initialised scratch buffers, one per (device, purpose), grown on demand.

    A buffer that was handed out once is NEVER freed or moved: a CUDA graph captured earlier keeps
    launching kernels on its address, so when a later call needs more, the old buffer is retired to
    ``_retired`` (kept alive for the life of the process) and a larger one takes its place for new
    calls.  In practice the first call of a model sizes the buffer and it never grows.

    Every decode call on a device shares one buffer: calls must be ordered on ONE stream (or inside
    one graph).  A caller that runs attention on several streams of one device passes its own
    ``workspace=`` tensor per stream to the ops instead.  (The e4m3 append scratch is not kept here:
    its contents are tied to one pool's geometry, so every ``KVPool`` owns its own.)"""

    def __init__(self):
        self._live: dict = {}
        self._retired: list = []

    def get(self, device, purpose: str, nbytes: int) -> torch.Tensor:
        key = (device.index, purpose)
        buf = self._live.get(key)
        if buf is None or buf.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("infer_b200: scratch memory has to be sized before a stream capture: "
                                   "call the op once eagerly first (the reference's capture loop does)")
            if buf is not None:
                self._retired.append(buf)
            buf = self._live[key] = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        return buf

    def clear(self):
        self._live.clear()
        self._retired.clear()


_SCRATCH = _Scratch()


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


class KVPool:
    """Handle on a pair of page pools ``[num_blocks, block_size, Hkv, 128]`` (bf16, or uint8
    holding e4m3 bytes together with fp32 ``[num_blocks, Hkv]`` scales).  Owns no memory and
    keeps no reference to the tensors (the caller keeps them alive, as the reference's runner
    does with ``self.kv_cache``); carries the TMA descriptors built once by the library."""

    def __init__(self, k_cache, v_cache, k_scale=None, v_scale=None):
        for t in (k_cache, v_cache):
            if not (t.is_cuda and t.dim() == 4 and t.is_contiguous()):
                raise ValueError("pools must be contiguous CUDA tensors [num_blocks, block_size, Hkv, head_dim]")
        if k_cache.shape != v_cache.shape or k_cache.dtype != v_cache.dtype:
            raise ValueError("k and v pools must agree in shape and dtype")
        fp8 = k_cache.dtype in (torch.uint8, torch.float8_e4m3fn)
        if not fp8 and k_cache.dtype != torch.bfloat16:
            raise ValueError("pools must be bf16 or e4m3 bytes")
        if fp8:
            nb, _, hkv, _ = k_cache.shape
            for s in (k_scale, v_scale):
                if s is None or s.dtype != torch.float32 or tuple(s.shape) != (nb, hkv) or not s.is_contiguous():
                    raise ValueError("e4m3 pools need contiguous fp32 scales [num_blocks, Hkv]")
        # The handle only borrows the tensors' memory (addresses and geometry): it keeps no
        # reference, so a cached handle never pins gigabytes of pool memory.
        self.fp8 = fp8
        self.num_blocks, self.block_size, self.n_kv_heads, self.head_dim = k_cache.shape
        self.device = k_cache.device
        lib = _lib.load()
        handle = C.c_void_p()
        with _on_device(self.device):
            rc = lib.infer_kv_pool_create(C.byref(handle), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale),
                                          self.num_blocks, self.block_size, self.n_kv_heads, self.head_dim,
                                          _lib.KV_E4M3 if fp8 else _lib.KV_BF16)
        _lib.check(rc, "infer_kv_pool_create")
        self.handle = handle
        self._decode_ws_bytes: dict = {}      # n_q_heads -> bytes, asked of the library once
        # e4m3 append scratch: its layout follows the pool's geometry and every call leaves it in the state
        # the next call on the SAME pool expects, so each pool owns one (sized here, never re-allocated)
        self.append_ws_bytes = lib.infer_kv_append_workspace_bytes(handle) if fp8 else 0
        self.append_ws = torch.zeros(self.append_ws_bytes, dtype=torch.uint8, device=self.device) if fp8 else None

    def decode_workspace_bytes(self, batch: int, n_q_heads: int) -> int:
        need = self._decode_ws_bytes.get(n_q_heads)
        if need is None:
            need = self._decode_ws_bytes[n_q_heads] = _lib.load().infer_paged_decode_workspace_bytes(
                self.handle, batch, n_q_heads)
        return need

    def __del__(self):
        h = getattr(self, "handle", None)
        if h and _lib is not None and getattr(_lib, "_lib", None) is not None:   # not at interpreter teardown
            _lib._lib.infer_kv_pool_destroy(h)
            self.handle = None


def pool_of(k_cache, v_cache, k_scale=None, v_scale=None) -> KVPool:
    """Pool handle for these cache tensors, created on first use (one per layer in practice)."""
    key = (k_cache.data_ptr(), v_cache.data_ptr(), tuple(k_cache.shape), k_cache.dtype,
           k_scale.data_ptr() if k_scale is not None else 0, v_scale.data_ptr() if v_scale is not None else 0)
    # A handle is valid for any tensor with the same addresses, shape and dtype, whatever Python
    # object presents them (a layer view sliced again every step, or new memory at an old address).
    pool = _POOLS.get(key)
    if pool is None:
        pool = _POOLS[key] = KVPool(k_cache, v_cache, k_scale, v_scale)
    return pool


def release_pools():
    """Forgets every pool handle and scratch buffer (only when no captured graph still uses them)."""
    _POOLS.clear()
    _SCRATCH.clear()


# --------------------------------------------------------------------------- append
def store_kvcache(key, value, k_cache, v_cache, slot_mapping, k_scale=None, v_scale=None, workspace=None):
    """``workspace`` (e4m3 pools only): a zero-initialised uint8 tensor of ``pool.append_ws_bytes``
    that this caller reserves for its own stream and this pool; by default the pool's own scratch is
    used (appends to one pool must then be ordered on one stream)."""
    n, num_heads, head_dim = key.shape
    d = num_heads * head_dim
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == head_dim and value.stride(1) == head_dim
    assert k_cache.stride(1) == d and v_cache.stride(1) == d
    assert slot_mapping.numel() == n
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16:
        raise RuntimeError("store_kvcache: key/value must be bf16")
    if slot_mapping.dtype != torch.int32 or not slot_mapping.is_cuda:
        raise RuntimeError("store_kvcache: slot_mapping must be an int32 CUDA tensor")
    if n == 0:
        return
    pool = pool_of(k_cache, v_cache, k_scale, v_scale)
    lib = _lib.load()
    # the pitch of a single row is meaningless (torch may report any stride for a size-1 dim)
    k_pitch = key.stride(0) if n > 1 else d
    v_pitch = value.stride(0) if n > 1 else d
    ws, ws_bytes = None, 0
    if pool.fp8:
        ws_bytes = pool.append_ws_bytes
        ws = workspace if workspace is not None else pool.append_ws
    with _on_device(pool.device):
        rc = lib.infer_kv_append(pool.handle, _ptr(key), _ptr(value), k_pitch, v_pitch,
                                 _ptr(slot_mapping), n, _ptr(ws), ws_bytes, _stream())
    _lib.check(rc, "store_kvcache")


def qk_norm_rope_append(q, k, v, q_norm_weight, k_norm_weight, eps, positions, cos_sin_cache, k_cache, v_cache,
                        slot_mapping, q_out=None):
    """Fused per-head RMSNorm (q, k) + NeoX rotary embedding (q, k) + KV append, one kernel.

    Replaces, for the attention block of the reference model (infer/models/Qwen3.py:112-131):
    ``q = q_norm(q); k = k_norm(k); rotary_emb(positions, q, k); store_kvcache(k, v, ...)``.
    q, k, v are ``[T, H, 128]`` views (column slices of the fused qkv output are fine);
    returns the normalised, rotated q as a contiguous ``[T, Hq, 128]`` tensor (or writes it into
    ``q_out``, which may be ``q``)."""
    t, hq, d = q.shape
    for name, x in (("q", q), ("k", k), ("v", v)):
        if x.dtype != torch.bfloat16 or x.stride(-1) != 1 or x.stride(1) != d:
            raise RuntimeError(f"qk_norm_rope_append: {name} must be bf16 [T, H, 128] with contiguous heads")
    if positions.dtype != torch.int64 or slot_mapping.dtype != torch.int32:
        raise RuntimeError("qk_norm_rope_append: positions must be int64 and slot_mapping int32")
    if cos_sin_cache.dtype != torch.bfloat16 or cos_sin_cache.shape[-1] != d or not cos_sin_cache.is_contiguous():
        raise RuntimeError("qk_norm_rope_append: cos_sin_cache must be contiguous bf16 [max_position, 128]")
    if q_out is None:
        q_out = torch.empty(t, hq, d, dtype=q.dtype, device=q.device)
    if t == 0:
        return q_out
    pool = pool_of(k_cache, v_cache)
    pitch = lambda x: x.stride(0) if t > 1 else x.shape[1] * d
    lib = _lib.load()
    with _on_device(pool.device):
        rc = lib.infer_qk_norm_rope_append(pool.handle, _ptr(q_out), pitch(q_out), _ptr(q), _ptr(k), _ptr(v), pitch(q),
                                           pitch(k), pitch(v), _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps),
                                           _ptr(positions), _ptr(cos_sin_cache), cos_sin_cache.shape[0],
                                           _ptr(slot_mapping), t, hq, _stream())
    _lib.check(rc, "qk_norm_rope_append")
    return q_out


# --------------------------------------------------------------------------- decode
def paged_attn_decode(q, k_cache, v_cache, cache_seqlens, block_table, softmax_scale,
                      out=None, k_scale=None, v_scale=None, workspace=None):
    """q [B, Hq, 128] (or [B, 1, Hq, 128] as the reference passes it) -> same shape.

    ``q`` and ``out`` may also be pinned host tensors: the kernel then reads the queries from, and writes the
    output rows straight into, host memory (a pinned tensor's address is valid on the device), which saves
    the separate copies of a host-fed step; pass ``out`` explicitly in that case.

    ``workspace``: a zero-initialised uint8 tensor of at least
    ``pool.decode_workspace_bytes(B, Hq)`` bytes reserved for this caller's stream; by default the
    per-device scratch is used (see ``_Scratch``: one stream per device)."""
    shape = q.shape
    q3 = q.reshape(shape[0], shape[-2], shape[-1])
    if q3.dtype != torch.bfloat16 or not q3.is_contiguous():
        raise RuntimeError("paged_attn_decode: q must be contiguous bf16")
    for name, t in (("q", q3), ("out", out)):
        if t is not None and not t.is_cuda and not t.is_pinned():
            raise RuntimeError(f"paged_attn_decode: {name} must live on the GPU or in pinned host memory")
    for name, t in (("cache_seqlens", cache_seqlens), ("block_table", block_table)):
        if t.dtype != torch.int32 or not t.is_cuda:
            raise RuntimeError(f"paged_attn_decode: {name} must be an int32 CUDA tensor")
    if block_table.stride(-1) != 1:
        raise RuntimeError("paged_attn_decode: block_table rows must be contiguous")
    pool = pool_of(k_cache, v_cache, k_scale, v_scale)
    o = torch.empty(q3.shape, dtype=q3.dtype, device=pool.device) if out is None else out.view(q3.shape)
    lib = _lib.load()
    b, hq, _ = q3.shape
    ws = workspace if workspace is not None else _SCRATCH.get(pool.device, "decode", pool.decode_workspace_bytes(b, hq))
    with _on_device(pool.device):
        rc = _call_decode(lib, pool.handle, _ptr(o), _ptr(q3), _ptr(cache_seqlens), _ptr(block_table),
                          block_table.stride(0), b, hq, float(softmax_scale), _ptr(ws), ws.numel(), _stream())
        _lib.check(rc, "paged_attn_decode")
        if _CHECK and not torch.cuda.is_current_stream_capturing():
            _lib.check(lib.infer_paged_decode_status(_ptr(ws), _stream()), "paged_attn_decode (device status)")
    return o.view(shape)


def paged_attn_decode_append(q, key, value, k_cache, v_cache, cache_seqlens, block_table, softmax_scale,
                             out=None, workspace=None):
    """``store_kvcache(key, value, ...)`` and ``paged_attn_decode(q, ...)`` of one decode step in ONE launch
    (bf16 pools; the two calls of infer/ops/attention.py:109 and :117-121).  ``key`` / ``value`` are the step's
    new rows ``[B, Hkv, 128]`` (column slices of a fused qkv output are fine), row b belonging to position
    ``cache_seqlens[b] - 1`` of sequence b; the slot is read off ``block_table``, so no ``slot_mapping`` is
    needed.  The pools end up as after ``store_kvcache``.  ``q``, ``key``, ``value`` and ``out`` may be pinned
    host tensors (see ``paged_attn_decode``)."""
    shape = q.shape
    q3 = q.reshape(shape[0], shape[-2], shape[-1])
    if q3.dtype != torch.bfloat16 or not q3.is_contiguous():
        raise RuntimeError("paged_attn_decode_append: q must be contiguous bf16")
    b, hq, d = q3.shape
    for name, t in (("key", key), ("value", value)):
        if t.dtype != torch.bfloat16 or t.dim() != 3 or t.shape[0] != b or t.stride(-1) != 1 or t.stride(1) != d:
            raise RuntimeError(f"paged_attn_decode_append: {name} must be bf16 [B, Hkv, 128] with contiguous heads")
    for name, t in (("q", q3), ("key", key), ("value", value), ("out", out)):
        if t is not None and not t.is_cuda and not t.is_pinned():
            raise RuntimeError(f"paged_attn_decode_append: {name} must live on the GPU or in pinned host memory")
    for name, t in (("cache_seqlens", cache_seqlens), ("block_table", block_table)):
        if t.dtype != torch.int32 or not t.is_cuda:
            raise RuntimeError(f"paged_attn_decode_append: {name} must be an int32 CUDA tensor")
    pool = pool_of(k_cache, v_cache)
    if pool.fp8:
        raise RuntimeError("paged_attn_decode_append: bf16 pools only (store_kvcache + paged_attn_decode for e4m3 pools)")
    if key.shape[1] != pool.n_kv_heads or value.shape != key.shape:
        raise RuntimeError("paged_attn_decode_append: key / value head count differs from the pool's")
    o = torch.empty(q3.shape, dtype=q3.dtype, device=pool.device) if out is None else out.view(q3.shape)
    lib = _lib.load()
    row = key.shape[1] * d
    k_pitch = key.stride(0) if b > 1 else row
    v_pitch = value.stride(0) if b > 1 else row
    ws = workspace if workspace is not None else _SCRATCH.get(pool.device, "decode", pool.decode_workspace_bytes(b, hq))
    with _on_device(pool.device):
        rc = lib.infer_paged_decode_append(pool.handle, _ptr(o), _ptr(q3), _ptr(key), _ptr(value), k_pitch, v_pitch,
                                           _ptr(cache_seqlens), _ptr(block_table), block_table.stride(0), b, hq,
                                           float(softmax_scale), _ptr(ws), ws.numel(), _stream())
        _lib.check(rc, "paged_attn_decode_append")
        if _CHECK and not torch.cuda.is_current_stream_capturing():
            _lib.check(lib.infer_paged_decode_status(_ptr(ws), _stream()), "paged_attn_decode_append (device status)")
    return o.view(shape)


# --------------------------------------------------------------------------- prefill
def paged_attn_prefill(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                       softmax_scale, block_table, out=None):
    """q [total_q, Hq, 128]; keys come from the pools through block_table; causal,
    bottom-right aligned (the flash_attn_varlen_func convention)."""
    if q.dtype != torch.bfloat16 or not q.is_contiguous() or q.dim() != 3:
        raise RuntimeError("paged_attn_prefill: q must be contiguous bf16 [total_q, Hq, 128]")
    for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k), ("block_table", block_table)):
        if t.dtype != torch.int32 or not t.is_cuda:
            raise RuntimeError(f"paged_attn_prefill: {name} must be an int32 CUDA tensor")
    pool = pool_of(k_cache, v_cache)
    o = torch.empty_like(q) if out is None else out
    lib = _lib.load()
    with _on_device(pool.device):
        rc = _call_prefill(lib, pool.handle, _ptr(o), _ptr(q), q.shape[0], _ptr(cu_seqlens_q), _ptr(cu_seqlens_k),
                                     _ptr(block_table), block_table.stride(0), cu_seqlens_q.numel() - 1,
                                     int(max_seqlen_q), int(max_seqlen_k), q.shape[1], float(softmax_scale),
                                     _stream())
        _lib.check(rc, "paged_attn_prefill")
        _check_prefill_status(lib, "paged_attn_prefill")
    return o


def _check_prefill_status(lib, what):
    """With INFER_B200_CHECK=1 (and outside stream capture): synchronise and raise if a bounded
    wait inside the prefill kernel ran out."""
    if _CHECK and not torch.cuda.is_current_stream_capturing():
        _lib.check(lib.infer_prefill_status(_stream()), f"{what} (device status)")


def flash_attn_prefill(Q, K, V, O):
    """Dense causal attention, Q/O [B, Hq, S, 128], K/V [B, Hkv, S, 128]; writes O."""
    for t in (Q, K, V, O):
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_cuda or t.dim() != 4:
            raise RuntimeError("flash_attn_prefill: tensors must be contiguous bf16 CUDA [B, H, S, 128]")
    if Q.shape[-1] != 128 or K.shape != V.shape or O.shape != Q.shape or K.shape[2] != Q.shape[2]:
        raise RuntimeError("flash_attn_prefill: shape mismatch")
    lib = _lib.load()
    with _on_device(Q.device):
        rc = _call_dense(lib, _ptr(Q), _ptr(K), _ptr(V), _ptr(O), Q.shape[0], Q.shape[1], K.shape[1],
                                          Q.shape[2], _stream())
        _lib.check(rc, "flash_attn_prefill")
        _check_prefill_status(lib, "flash_attn_prefill")


# --------------------------------------------------------------------------- torch.ops._C
_REGISTERED = False


def register_torch_ops():
    """Registers the ops under the ``_C`` namespace the reference uses
    (TORCH_LIBRARY(_C), src/bindings.cpp:4-37), CUDA dispatch key only."""
    global _REGISTERED, _torch_lib
    if _REGISTERED:
        return
    lib = torch.library.Library("_C", "FRAGMENT")
    lib.define("flash_attn_prefill(Tensor Q, Tensor K, Tensor V, Tensor! O) -> ()")
    lib.define("store_kvcache(Tensor key, Tensor value, Tensor! k_cache, Tensor! v_cache, Tensor slot_mapping) -> ()")
    lib.define("paged_attn_decode(Tensor! out, Tensor q, Tensor k_cache, Tensor v_cache, Tensor cache_seqlens, "
               "Tensor block_table, float softmax_scale) -> ()")
    lib.define("paged_attn_prefill(Tensor! out, Tensor q, Tensor k_cache, Tensor v_cache, Tensor cu_seqlens_q, "
               "Tensor cu_seqlens_k, int max_seqlen_q, int max_seqlen_k, float softmax_scale, Tensor block_table) -> ()")
    lib.impl("flash_attn_prefill", lambda Q, K, V, O: flash_attn_prefill(Q, K, V, O), "CUDA")
    lib.impl("store_kvcache", lambda k, v, kc, vc, sm: store_kvcache(k, v, kc, vc, sm), "CUDA")
    lib.impl("paged_attn_decode",
             lambda out, q, kc, vc, sl, bt, sc: (paged_attn_decode(q, kc, vc, sl, bt, sc, out=out), None)[1], "CUDA")
    lib.impl("paged_attn_prefill",
             lambda out, q, kc, vc, cq, ck, mq, mk, sc, bt:
             (paged_attn_prefill(q, kc, vc, cq, ck, mq, mk, sc, bt, out=out), None)[1], "CUDA")
    _torch_lib = lib
    _REGISTERED = True
