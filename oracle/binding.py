"""ctypes binding of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg import this
module; the product package never does.  The shared object is built from
relux_oracle.cpp by `make -C oracle` (done on demand here).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librelux_oracle.so")

FAITHFUL, INTENDED = 0, 1
FLAG_MLA_BF16_CACHE = 1

MHA_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float),
                       C.POINTER(C.c_float), C.POINTER(C.c_float))
LAYER_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float))
MLA_HOOK = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float),
                       C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float))


class ModelCfg(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("dModel", C.c_int32), ("numHeads", C.c_int32), ("numKVHeads", C.c_int32),
                ("numLayers", C.c_int32), ("dFF", C.c_int32), ("maxSeqLen", C.c_int32), ("ropeBase", C.c_float),
                ("causal", C.c_int32), ("swiglu", C.c_int32), ("mla", C.c_int32), ("dC", C.c_int32), ("dHR", C.c_int32)]


def build(force=False):
    srcs = [os.path.join(_HERE, n) for n in ("relux_oracle.cpp", "relux_oracle_sampling.inc")]
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(s) for s in srcs):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        L = _lib
        L.ro_bf16_from_f32.restype = C.c_uint16
        L.ro_bf16_from_f32.argtypes = [C.c_float]
        L.ro_f32_from_bf16.restype = C.c_float
        L.ro_f32_from_bf16.argtypes = [C.c_uint16]
        L.ro_fastexp32.restype = C.c_float
        L.ro_fastexp32.argtypes = [C.c_float]
        L.ro_gelu.restype = C.c_float
        L.ro_gelu.argtypes = [C.c_float]
        for n in ("ro_rope_new", "ro_kvcache_new", "ro_kvcache_new_sized", "ro_mlacache_new", "ro_model_new"):
            getattr(L, n).restype = C.c_void_p
        L.ro_rope_new.argtypes = [C.c_int, C.c_float, C.c_int]
        L.ro_rope_cos.restype = C.POINTER(C.c_float)
        L.ro_rope_sin.restype = C.POINTER(C.c_float)
        L.ro_kvcache_view_shape.restype = C.c_int64
        L.ro_model_weight_count.restype = C.c_int64
    return _lib


def _p(a, t=None):
    if a is None:
        return None
    return a.ctypes.data_as(C.c_void_p)


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- scalar / slice helpers -------------------------------------------------
def bf16_from_f32(a):
    a = f32(a)
    out = np.empty(a.shape, np.uint16)
    lib().ro_bf16_slice_from_f32(_p(a), _p(out), C.c_int64(a.size))
    return out


def f32_from_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().ro_f32_slice_from_bf16(_p(a), _p(out), C.c_int64(a.size))
    return out


def bf16_from_f64(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    out = np.empty(a.shape, np.uint16)
    lib().ro_bf16_slice_from_f64(_p(a), _p(out), C.c_int64(a.size))
    return out


def fastexp32(x):
    return float(lib().ro_fastexp32(C.c_float(x)))


def softmax_rows(m):
    m = f32(m).copy()
    lib().ro_softmax_rows(_p(m), C.c_int(m.shape[0]), C.c_int(m.shape[1]))
    return m


def matmul(a, b):
    a, b = f32(a), f32(b)
    out = np.empty((a.shape[0], b.shape[1]), np.float32)
    lib().ro_matmul(_p(out), _p(a), _p(b), a.shape[0], a.shape[1], b.shape[1])
    return out


def matmul_transb(a, b):
    a, b = f32(a), f32(b)
    out = np.empty((a.shape[0], b.shape[0]), np.float32)
    lib().ro_matmul_transb(_p(out), _p(a), _p(b), a.shape[0], a.shape[1], b.shape[0])
    return out


def rmsnorm(x, eps):
    x = f32(x)
    D = x.shape[-1]
    out = np.empty_like(x)
    lib().ro_rmsnorm(_p(out), _p(x), C.c_int(x.size // D), C.c_int(D), C.c_float(eps))
    return out


def greedy(logits):
    l = f32(logits)
    return int(lib().ro_greedy(_p(l), C.c_int(l.size)))


# ---- RoPE -------------------------------------------------------------------
class Rope:
    def __init__(self, head_dim, base, max_seq_len):
        self.h = lib().ro_rope_new(head_dim, C.c_float(base), max_seq_len)
        if not self.h:
            raise ValueError("NewRotaryEmbedding: invalid arguments (the reference panics)")
        self.head_dim = head_dim

    def __del__(self):
        if getattr(self, "h", None):
            lib().ro_rope_free(C.c_void_p(self.h))

    @property
    def max_seq_len(self):
        return lib().ro_rope_max_seq_len(C.c_void_p(self.h))

    def cos(self):
        n = self.max_seq_len * self.head_dim // 2
        return np.ctypeslib.as_array(lib().ro_rope_cos(C.c_void_p(self.h)), (n,)).copy()

    def sin(self):
        n = self.max_seq_len * self.head_dim // 2
        return np.ctypeslib.as_array(lib().ro_rope_sin(C.c_void_p(self.h)), (n,)).copy()

    def extend(self, new_max):
        if lib().ro_rope_extend(C.c_void_p(self.h), new_max):
            raise ValueError("ExtendMaxSeqLen: newMax must exceed current (the reference panics)")

    def apply(self, x, start_pos, intended_positions=False):
        x = f32(x)
        out = np.empty_like(x)
        rank1 = x.ndim == 1
        seq = 1 if rank1 else x.shape[-2]
        rc = lib().ro_rope_apply(C.c_void_p(self.h), _p(x), _p(out), C.c_int64(x.size // self.head_dim), seq,
                                 int(rank1), start_pos, int(intended_positions))
        if rc:
            raise IndexError("RotaryEmbedding.Apply: position >= maxSeqLen (the reference panics)")
        return out


# ---- KVCache ----------------------------------------------------------------
class KVCache:
    F32, BF16 = 0, 1

    def __init__(self, num_layers, dtype, max_len=0, num_kv_heads=0, head_dim=0):
        if max_len > 0:
            self.h = lib().ro_kvcache_new_sized(num_layers, max_len, num_kv_heads, head_dim, dtype)
        else:
            self.h = lib().ro_kvcache_new(num_layers, dtype)
        if not self.h:
            raise ValueError("NewKVCache: invalid arguments (the reference panics)")
        self.dtype = dtype

    def __del__(self):
        if getattr(self, "h", None):
            lib().ro_kvcache_free(C.c_void_p(self.h))

    def append(self, layer, k, v):
        k, v = f32(k), f32(v)
        if k.shape != v.shape:
            raise ValueError("KVCache.Append: K and V shape mismatch")
        shape = (C.c_int * k.ndim)(*k.shape)
        rc = lib().ro_kvcache_append(C.c_void_p(self.h), layer, _p(k), _p(v), shape, k.ndim)
        if rc:
            raise RuntimeError("KVCache.Append panic code %d" % rc)

    def total_len(self, layer):
        return lib().ro_kvcache_total_len(C.c_void_p(self.h), layer)

    def view(self, layer, raw_bf16=False):
        shape = (C.c_int * 8)()
        rank = C.c_int(0)
        n = lib().ro_kvcache_view_shape(C.c_void_p(self.h), layer, shape, C.byref(rank))
        if n < 0:
            raise IndexError("KVCache.View: layerIdx out of range")
        if rank.value == 0:
            return None, None
        shp = tuple(shape[i] for i in range(rank.value))
        if raw_bf16:
            k, v = np.empty(n, np.uint16), np.empty(n, np.uint16)
            lib().ro_kvcache_read_bf16(C.c_void_p(self.h), layer, _p(k), _p(v), C.c_int64(n))
        else:
            k, v = np.empty(n, np.float32), np.empty(n, np.float32)
            lib().ro_kvcache_read_f32(C.c_void_p(self.h), layer, _p(k), _p(v), C.c_int64(n))
        return k.reshape(shp), v.reshape(shp)

    def reset(self):
        lib().ro_kvcache_reset(C.c_void_p(self.h))


class MLACache:
    def __init__(self, num_layers, max_len, dC, dHR, round_bf16=False):
        self.h = lib().ro_mlacache_new(num_layers, max_len, dC, dHR, int(round_bf16))
        if not self.h:
            raise ValueError("NewMLACache: invalid arguments (the reference panics)")
        self.dC, self.dHR = dC, dHR

    def __del__(self):
        if getattr(self, "h", None):
            lib().ro_mlacache_free(C.c_void_p(self.h))

    def append(self, layer, new_c, new_kr):
        c, r = f32(new_c), f32(new_kr)
        rc = lib().ro_mlacache_append(C.c_void_p(self.h), layer, _p(c), C.c_int64(c.size), _p(r), C.c_int64(r.size),
                                      c.shape[-2])
        if rc:
            raise RuntimeError("MLACache.Append panic code %d" % rc)

    def total_len(self, layer):
        return lib().ro_mlacache_total_len(C.c_void_p(self.h), layer)

    def view(self, layer):
        t = self.total_len(layer)
        c, r = np.empty((1, t, self.dC), np.float32), np.empty((1, t, self.dHR), np.float32)
        lib().ro_mlacache_read(C.c_void_p(self.h), layer, _p(c), _p(r))
        return c, r

    def reset(self):
        lib().ro_mlacache_reset(C.c_void_p(self.h))


# ---- decoder model ----------------------------------------------------------
class Model:
    def __init__(self, cfg: ModelCfg, flat_weights_bf16):
        w = np.ascontiguousarray(flat_weights_bf16, dtype=np.uint16)
        need = lib().ro_model_weight_count(C.byref(cfg))
        if w.size != need:
            raise ValueError("flat weight buffer has %d elements, model needs %d" % (w.size, need))
        self.cfg = cfg
        self.h = lib().ro_model_new(C.byref(cfg), _p(w))
        if not self.h:
            raise ValueError("NewTransformer: invalid config")
        self._hooks = None

    def __del__(self):
        if getattr(self, "h", None):
            lib().ro_model_free(C.c_void_p(self.h))

    @staticmethod
    def weight_count(cfg):
        return int(lib().ro_model_weight_count(C.byref(cfg)))

    def set_mode(self, mode, flags=0):
        lib().ro_model_set_mode(C.c_void_p(self.h), mode, flags)

    def set_hooks(self, mha=None, mla=None):
        a = MHA_HOOK(mha) if mha else C.cast(None, MHA_HOOK)
        b = MLA_HOOK(mla) if mla else C.cast(None, MLA_HOOK)
        self._hooks = (a, b)  # keep alive
        lib().ro_model_set_hooks(C.c_void_p(self.h), a, b, None)

    def set_layer_hook(self, fn):
        """fn(user, layer, S, x_ptr, out_ptr) -> int replaces the whole cached attention layer forward."""
        h = LAYER_HOOK(fn) if fn else C.cast(None, LAYER_HOOK)
        self._layer_hook = h  # keep alive
        lib().ro_model_set_layer_hook(C.c_void_p(self.h), h)

    def begin(self):
        lib().ro_model_begin(C.c_void_p(self.h))

    def attention_forward(self, layer, x):
        """The attention module of `layer` alone (forwardCached on the session's caches): x [seq, dModel] -> [seq, dModel]."""
        x = f32(x)
        out = np.empty_like(x)
        rc = lib().ro_model_attention_forward(C.c_void_p(self.h), int(layer), _p(x), C.c_int(x.shape[0]), _p(out))
        if rc:
            raise RuntimeError("forwardCached failed with code %d" % rc)
        return out

    def forward(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((t.size, self.cfg.vocab), np.float32)
        rc = lib().ro_model_forward(C.c_void_p(self.h), _p(t), C.c_int(t.size), _p(out))
        if rc:
            raise RuntimeError("Transformer.Forward failed with code %d" % rc)
        return out

    def generate(self, prompt, max_new):
        t = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(t.size + max_new, np.int32)
        margins = np.empty(max_new, np.float32)
        ties = C.c_int(0)
        rc = lib().ro_model_generate(C.c_void_p(self.h), _p(t), C.c_int(t.size), C.c_int(max_new), _p(out), _p(margins),
                                     C.byref(ties))
        if rc:
            raise RuntimeError("Transformer.Generate failed with code %d" % rc)
        return out, margins, ties.value


# ---- standalone attention ops ----------------------------------------------
def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _u16(a):
    return np.ascontiguousarray(a, dtype=np.uint16)


def mla_attend(ckv, kr, ctx, qc, qr, W_UK, W_UV, scale, causal=True, absorbed=False, threads=0):
    """ckv [B,Tmax,dC] bf16 bits, kr [B,Tmax,dHR] bf16 bits, ctx [B], qc [B,S,H,Dh] f32, qr [B,S,H,dHR] f32."""
    ckv, kr, qc, qr, ctx = _u16(ckv), _u16(kr), f32(qc), f32(qr), _i32(ctx)
    W_UK, W_UV = _u16(W_UK), _u16(W_UV)
    B, Tmax, dC = ckv.shape
    _, S, H, Dh = qc.shape
    dHR = kr.shape[2]
    out = np.empty((B, S, H, Dh), np.float32)
    fn = lib().ro_mla_attend_absorbed if absorbed else lib().ro_mla_attend_decompress
    fn(B, S, H, Dh, dC, dHR, Tmax, _p(ctx), _p(ckv), _p(kr), _p(qc), _p(qr), _p(W_UK), _p(W_UV), C.c_float(scale),
       int(causal), _p(out), threads)
    return out


def gqa_attend(K, V, ctx, q, scale, causal=True, threads=0, reference_cost=False, capacity=0):
    """K,V [B,Tmax,Hkv,D] bf16 bits, ctx [B], q [B,S,H,D] f32 -> [B,S,H,D] f32."""
    K, V, q, ctx = _u16(K), _u16(V), f32(q), _i32(ctx)
    B, Tmax, Hkv, D = K.shape
    _, S, H, _ = q.shape
    out = np.empty((B, S, H, D), np.float32)
    if reference_cost:
        lib().ro_gqa_attend_reference_cost(B, S, H, Hkv, D, Tmax, max(capacity, Tmax), _p(ctx), _p(K), _p(V), _p(q),
                                           C.c_float(scale), int(causal), _p(out), threads)
    else:
        lib().ro_gqa_attend(B, S, H, Hkv, D, Tmax, _p(ctx), _p(K), _p(V), _p(q), C.c_float(scale), int(causal), _p(out),
                            threads)
    return out


def set_exact_exp(on):
    """Test-only: softmaxRows with libm exp instead of fastexp32 (see relux_oracle.cpp)."""
    lib().ro_set_exact_exp(int(bool(on)))


class exact_exp:
    def __enter__(self):
        set_exact_exp(True)

    def __exit__(self, *a):
        set_exact_exp(False)


def num_threads():
    return int(lib().ro_num_threads())


# ---- sampler and speculative accept step ------------------------------------
class SamplerCfg(C.Structure):
    """Sampler's fields (sampler.go:34-44) without the generator: draws are passed to each call."""
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("min_p", C.c_float),
                ("repeat_penalty", C.c_float), ("frequency_penalty", C.c_float), ("presence_penalty", C.c_float),
                ("repeat_window", C.c_int32)]


def sampler_cfg(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, frequency_penalty=0.0,
                presence_penalty=0.0, repeat_window=0):
    return SamplerCfg(temperature, top_k, top_p, min_p, repeat_penalty, frequency_penalty, presence_penalty, repeat_window)


def sampler_sample(cfg, logits, r, prev=None, return_probs=False):
    """Sampler.Sample (sampler.go:73-218) with the categorical draw r supplied."""
    l = f32(logits)
    pv = _i32(prev) if prev is not None and len(prev) else None
    probs = np.empty(l.size, np.float32)
    lib().ro_sampler_sample.restype = C.c_int
    tok = lib().ro_sampler_sample(C.byref(cfg), _p(l), C.c_int(l.size), _p(pv) if pv is not None else None,
                                  C.c_int(0 if pv is None else pv.size), C.c_float(r), _p(probs))
    return (int(tok), probs) if return_probs else int(tok)


def softmax_alloc(logits):
    """softmaxAlloc (speculative.go:346-368)."""
    l = f32(logits)
    out = np.empty_like(l)
    lib().ro_softmax_alloc(_p(l), C.c_int(l.size), _p(out))
    return out


def spec_accept(cfg, draft_tokens, draft_logits, target_logits, draws):
    """acceptPhase (speculative.go:211-253) for one sequence: draft_logits [k][V], target_logits [k+1][V],
    draws [k+1] consumed in the reference's order.  Returns (n_accepted, next_token, draws_used, accept_probs[k])."""
    dt = _i32(draft_tokens)
    dl, tl, u = f32(draft_logits), f32(target_logits), f32(draws)
    k, V = dl.shape
    assert tl.shape == (k + 1, V) and u.size >= k + 1
    nxt, used = C.c_int32(-1), C.c_int32(0)
    ap = np.full(k, np.nan, np.float32)
    lib().ro_spec_accept.restype = C.c_int
    n = lib().ro_spec_accept(C.byref(cfg), _p(dt), _p(dl), _p(tl), C.c_int(k), C.c_int(V), _p(u), C.byref(nxt),
                             C.byref(used), _p(ap))
    return int(n), int(nxt.value), int(used.value), ap


# ---- matmulBatched3D and the checkpoint -> relux weight layout ---------------------------------
def matmul_batched3d(a, w_bf16):
    """matmulBatched3D (internal/transformer/mha.go:759-785 -> nativeBackend.MatMulFloat32, internal/compute/native.go:175-187):
    a [M, K] float32 x w [K, N] bf16 bits -> [M, N] float32, one k-ascending unfused multiply-add chain per output."""
    a = f32(a)
    w = np.ascontiguousarray(w_bf16, dtype=np.uint16)
    out = np.empty((a.shape[0], w.shape[1]), np.float32)
    fn = lib().ro_matmul_batched3d
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]
    fn.restype = None
    fn(_p(out), _p(a), _p(w), 1, a.shape[0], a.shape[1], w.shape[1])
    return out


def import_mla_weights(d_model, num_heads, nope_dim, rope_dim, v_dim, dc, q_proj=None, kv_a_proj_with_mqa=None, kv_b_proj=None,
                       o_proj=None, q_pe_proj=None, k_pe_proj=None, fused_rope=False):
    """Restatement (numpy) of what the reference's loader is specified to do with a DeepSeek MLA layer: every tensor is
    stored [out, in] and marked Transpose: true (internal/loader/mapper.go:43-49, 139-180), converted to bf16 with
    BF16FromF32 (loader.go:239-281, 394-404); kv_b_proj holds, per head, the nope rows of W_UK followed by the v rows of W_UV
    (mapper.go:146-152).  Sources: float32 arrays or uint16 bf16 bits.  Returns a dict of uint16 arrays in relux's [in, out]
    layout, keyed like relux_mla_layer_weights."""
    def bits(x):
        x = np.ascontiguousarray(x)
        return x if x.dtype == np.uint16 else bf16_from_f32(x)

    H, out = num_heads, {}
    if q_proj is not None:
        per = nope_dim + (rope_dim if fused_rope else 0)
        q = bits(q_proj).reshape(H, per, d_model)
        out["w_q"] = np.ascontiguousarray(q[:, :nope_dim].reshape(H * nope_dim, d_model).T)
        if fused_rope:
            out["w_qr"] = np.ascontiguousarray(q[:, nope_dim:].reshape(H * rope_dim, d_model).T)
    if kv_a_proj_with_mqa is not None:
        a = bits(kv_a_proj_with_mqa)
        out["w_dkv"] = np.ascontiguousarray(a[:dc].T)
        if fused_rope:
            out["w_kr"] = np.ascontiguousarray(a[dc:dc + rope_dim].T)
    if q_pe_proj is not None:
        out["w_qr"] = np.ascontiguousarray(bits(q_pe_proj).T)
    if k_pe_proj is not None:
        out["w_kr"] = np.ascontiguousarray(bits(k_pe_proj).T)
    if kv_b_proj is not None:
        b = bits(kv_b_proj).reshape(H, nope_dim + v_dim, dc)
        out["w_uk"] = np.ascontiguousarray(b[:, :nope_dim].reshape(H * nope_dim, dc).T)
        out["w_uv"] = np.ascontiguousarray(b[:, nope_dim:].reshape(H * v_dim, dc).T)
    if o_proj is not None:
        out["w_o"] = np.ascontiguousarray(bits(o_proj).T)
    return out
