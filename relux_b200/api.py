"""Host-side mirror of relux's KV-cache and cached-attention interface over librelux_cuda.so.

Two levels:

* `Pool` -- the batched, paged interface the CUDA library is built around (many sequences, page tables,
  append / decode / verify on host or device arrays).
* `KVCache`, `MLACache` -- single-sequence objects with the reference's own method set
  (Append / View / TotalLen / Reset / DType; internal/transformer/kvcache.go:169-388,
  internal/transformer/mla_cache.go:118-241) plus `attend`, the replacement for the attention loops of
  MHA.forwardCached (mha.go:292-348) and MLA.forwardCached (mla.go:317-377).  Misuse that panics in the
  reference raises here with the same wording.

Arrays are numpy; bf16 travels as uint16 bit patterns.  Nothing here computes on the CPU: every
operation is a call into the shared library.
"""
import ctypes as C

import os

import numpy as np

from . import lib as L


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, DeviceBuffer):
        return a.ptr
    if isinstance(a, int):
        return a
    return a.ctypes.data


def _mem(a):
    return L.MEM_DEVICE if isinstance(a, (DeviceBuffer, int)) else L.MEM_HOST


def _dtype_flag(a, explicit=None):
    if explicit is not None:
        return explicit
    if isinstance(a, DeviceBuffer):
        return a.dtype_flag
    if a.dtype == np.float32:
        return L.DTYPE_F32
    if a.dtype == np.uint16:
        return L.DTYPE_BF16
    raise TypeError("arrays must be float32 or uint16 (bf16 bits), got %s" % a.dtype)


class Device:
    """One GPU.  Mirrors compute.NewComputeBackend's role for this path (internal/compute/factory.go:32-85):
    it either opens a usable sm_100 device or raises -- there is no silent native fallback."""

    def __init__(self, index=0):
        self.lib = L.load()
        h = C.c_void_p()
        L.check(self.lib.relux_cuda_device_open(index, C.byref(h)))
        self.h = h
        self.index = index

    def close(self):
        if self.h:
            L.check(self.lib.relux_cuda_device_close(self.h))
            self.h = None

    def sync(self):
        L.check(self.lib.relux_cuda_sync(self.h))

    def info(self):
        name = C.create_string_buffer(256)
        sm = C.c_int32()
        mem = C.c_int64()
        L.check(self.lib.relux_cuda_device_info(self.h, name, 256, C.byref(sm), C.byref(mem)))
        return {"name": name.value.decode(), "sm_count": sm.value, "total_mem": mem.value}

    def launch_count(self):
        n = C.c_int64()
        L.check(self.lib.relux_cuda_launch_count(self.h, C.byref(n)))
        return n.value

    def alloc(self, nbytes, dtype_flag=L.DTYPE_BF16):
        return DeviceBuffer(self, nbytes, dtype_flag)

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        b = DeviceBuffer(self, arr.nbytes, L.DTYPE_F32 if arr.dtype == np.float32 else L.DTYPE_BF16)
        b.upload(arr)
        return b

    def pinned(self, shape, dtype):
        """A numpy array over pinned host memory (freed when the returned holder is closed)."""
        return PinnedArray(self, shape, dtype)

    def flush_l2(self):
        L.check(self.lib.relux_cuda_flush_l2(self.h))

    def event(self):
        return Event(self)


class Event:
    def __init__(self, dev):
        self.dev = dev
        self.h = C.c_void_p()
        L.check(dev.lib.relux_cuda_event_create(dev.h, C.byref(self.h)))

    def record(self):
        L.check(self.dev.lib.relux_cuda_event_record(self.dev.h, self.h))

    def elapsed_ms(self, later):
        ms = C.c_float()
        L.check(self.dev.lib.relux_cuda_event_elapsed_ms(self.dev.h, self.h, later.h, C.byref(ms)))
        return ms.value

    def close(self):
        if self.h:
            self.dev.lib.relux_cuda_event_destroy(self.dev.h, self.h)
            self.h = None


class DeviceBuffer:
    def __init__(self, dev, nbytes, dtype_flag=L.DTYPE_BF16):
        self.dev = dev
        self.nbytes = int(nbytes)
        self.dtype_flag = dtype_flag
        p = C.c_void_p()
        L.check(dev.lib.relux_cuda_dev_alloc(dev.h, self.nbytes, C.byref(p)))
        self.ptr = p.value or 0

    def upload(self, arr, offset=0):
        arr = np.ascontiguousarray(arr)
        assert offset + arr.nbytes <= self.nbytes
        L.check(self.dev.lib.relux_cuda_h2d(self.dev.h, self.ptr + offset, arr.ctypes.data, arr.nbytes))
        self.dev.sync()  # the source may be pageable and die after this call

    def download(self, shape, dtype, offset=0):
        out = np.empty(shape, dtype)
        assert offset + out.nbytes <= self.nbytes
        L.check(self.dev.lib.relux_cuda_d2h(self.dev.h, out.ctypes.data, self.ptr + offset, out.nbytes))
        return out

    def zero(self):
        L.check(self.dev.lib.relux_cuda_memset(self.dev.h, self.ptr, 0, self.nbytes))

    def free(self):
        if self.ptr:
            L.check(self.dev.lib.relux_cuda_dev_free(self.dev.h, self.ptr))
            self.ptr = 0


class PinnedArray:
    def __init__(self, dev, shape, dtype):
        self.dev = dev
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        L.check(dev.lib.relux_cuda_host_alloc(dev.h, n, C.byref(p)))
        self.ptr = p.value
        buf = (C.c_char * n).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=dtype).reshape(shape)

    def close(self):
        if self.ptr:
            self.array = None
            L.check(self.dev.lib.relux_cuda_host_free(self.dev.h, self.ptr))
            self.ptr = None


class Pool:
    """Paged bf16 KV pool on one device (see relux_pool_create in include/relux_cuda.h)."""

    def __init__(self, dev, kind, num_layers, num_pages, page_tokens=64, max_seqs=1, max_pages_per_seq=None, dC=0, dHR=0,
                 num_kv_heads=0, head_dim=0, reference_compat=False):
        self.dev = dev
        self.lib = dev.lib
        if max_pages_per_seq is None:
            max_pages_per_seq = num_pages
        prm = L.PoolParams(kind=kind, num_layers=num_layers, num_pages=num_pages, page_tokens=page_tokens, max_seqs=max_seqs,
                           max_pages_per_seq=max_pages_per_seq, mla_dc=dC, mla_dhr=dHR, gqa_num_kv_heads=num_kv_heads,
                           gqa_head_dim=head_dim, flags=L.POOL_FLAG_REFERENCE_COMPAT if reference_compat else 0)
        self.prm = prm
        self.kind = kind
        h = C.c_void_p()
        L.check(self.lib.relux_pool_create(dev.h, C.byref(prm), C.byref(h)))
        self.h = h
        self._keep = []

    def destroy(self):
        if self.h:
            L.check(self.lib.relux_pool_destroy(self.h))
            self.h = None

    def reset(self):
        L.check(self.lib.relux_pool_reset(self.h))

    def set_tables(self, table, ctx_len=None):
        table = np.ascontiguousarray(table, dtype=np.int32)
        cl = None if ctx_len is None else np.ascontiguousarray(ctx_len, dtype=np.int32)
        L.check(self.lib.relux_pool_set_tables(self.h, table.ctypes.data, table.shape[0], table.shape[1], _ptr(cl)))

    def seq_alloc(self, max_tokens):
        s = C.c_int32()
        L.check(self.lib.relux_seq_alloc(self.h, max_tokens, C.byref(s)))
        return s.value

    def seq_free(self, seq):
        L.check(self.lib.relux_seq_free(self.h, seq))

    def seq_extend(self, seq, max_tokens):
        """Grows a sequence made by seq_alloc to hold max_tokens rows (pages come from the pool's free list)."""
        L.check(self.lib.relux_seq_extend(self.h, seq, max_tokens))

    def seq_len(self, layer, seq):
        n = C.c_int32()
        L.check(self.lib.relux_seq_len(self.h, layer, seq, C.byref(n)))
        return n.value

    def set_len(self, layer, new_len, seq_ids=None):
        nl = np.ascontiguousarray(new_len, dtype=np.int32)
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        L.check(self.lib.relux_seq_set_len(self.h, layer, nl.size, _ptr(ids), nl.ctypes.data))

    def status(self):
        s = C.c_int32()
        L.check(self.lib.relux_pool_status(self.h, C.byref(s)))
        return s.value

    def read_rows(self, layer, seq, tok0, n):
        p = self.prm
        if self.kind == L.POOL_MLA:
            a, b = np.empty((n, p.mla_dc), np.uint16), np.empty((n, p.mla_dhr), np.uint16)
        else:
            a = np.empty((n, p.gqa_num_kv_heads, p.gqa_head_dim), np.uint16)
            b = np.empty_like(a)
        args = L.ReadRowsArgs(layer=layer, seq_id=seq, tok0=tok0, n_tokens=n, dst_a=a.ctypes.data, dst_b=b.ctypes.data)
        L.check(self.lib.relux_pool_read_rows(self.h, C.byref(args)))
        return a, b

    def wait_output(self, calls_back=0):
        """Blocks until the host output of a pipelined attention call has landed (0: the latest call, 1: the one before)."""
        L.check(self.lib.relux_pool_wait_output(self.h, int(calls_back)))

    def tune(self, knob, value):
        """Sets one tuning knob (L.TUNE_*); a negative value restores the built-in default."""
        L.check(self.lib.relux_pool_tune(self.h, int(knob), int(value)))

    def matmul(self, a, w, n, out=None, mode=L.ATTN_FAST):
        """C [M, N] float32 = a [M, K] float32 x w [K, N] bf16 on the device (ComputeBackend.MatMulFloat32 as
        matmulBatched3D calls it: mha.go:759-785).  a / out: numpy arrays or device buffers; w: device buffer."""
        if isinstance(a, DeviceBuffer):
            raise TypeError("matmul: pass a as a numpy array, or call the C entry point with explicit sizes")
        a = np.ascontiguousarray(a, dtype=np.float32)
        m, k = a.shape
        res = np.empty((m, n), np.float32) if out is None else out
        args = L.MatmulArgs(m=m, k=k, n=n, mode=mode, a=_ptr(a), a_mem=_mem(a), c_mem=_mem(res), b=_ptr(w), c=_ptr(res))
        L.check(self.lib.relux_matmul_f32_bf16(self.h, C.byref(args)))
        return res

    def import_mla_weights(self, d_model, num_heads, nope_dim, rope_dim, v_dim, dc, dst, q_proj=None, kv_a_proj_with_mqa=None,
                           kv_b_proj=None, o_proj=None, q_pe_proj=None, k_pe_proj=None, fused_rope=False):
        """Splits and transposes one layer's DeepSeek-style checkpoint tensors (numpy float32 or uint16 bf16 bits, all of
        one dtype) into the device buffers `dst` (dict w_q, w_qr, w_dkv, w_kr, w_uk, w_uv, w_o); see relux_mla_import_weights."""
        srcs = [x for x in (q_proj, kv_a_proj_with_mqa, kv_b_proj, o_proj, q_pe_proj, k_pe_proj) if x is not None]
        srcs = [np.ascontiguousarray(x) for x in srcs]
        dt = {_dtype_flag(x) for x in srcs}
        if len(dt) != 1:
            raise TypeError("import_mla_weights: sources must share one dtype")
        hold = {}

        def src(x):
            if x is None:
                return None
            x = np.ascontiguousarray(x)
            hold[id(x)] = x
            return x.ctypes.data

        w = L.MlaLayerWeights(**{k: _ptr(dst.get(k)) for k in ("w_q", "w_qr", "w_dkv", "w_kr", "w_uk", "w_uv", "w_o")})
        args = L.MlaImportArgs(d_model=d_model, num_heads=num_heads, nope_dim=nope_dim, rope_dim=rope_dim, v_dim=v_dim, dc=dc,
                               src_dtype=dt.pop(), src_mem=L.MEM_HOST, fused_rope=int(fused_rope), q_proj=src(q_proj),
                               kv_a_proj_with_mqa=src(kv_a_proj_with_mqa), kv_b_proj=src(kv_b_proj), o_proj=src(o_proj),
                               q_pe_proj=src(q_pe_proj), k_pe_proj=src(k_pe_proj), dst=C.pointer(w))
        L.check(self.lib.relux_mla_import_weights(self.h, C.byref(args)))

    def expand_kv(self, layer, n_seqs, num_heads, w_uk, w_uv, seq_ids=None, extra_tokens=0):
        """Cached MLA latents times W_UK / W_UV (relux_mla_expand_kv).  Returns (k, v, seq_base): k, v uint16 (bf16 bits)
        [num_heads][rows_total][128] host arrays, seq_base int32 [n_seqs + 1] (first row of every sequence)."""
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        rows = C.c_int64()
        args = L.MlaExpandArgs(layer=layer, n_seqs=n_seqs, seq_ids=_ptr(ids), extra_tokens=extra_tokens, num_heads=num_heads,
                               w_uk=_ptr(w_uk), w_uv=_ptr(w_uv), kv_out=None, seq_base=None, rows_total=0,
                               rows_total_out=C.pointer(rows))
        L.check(self.lib.relux_mla_expand_kv(self.h, C.byref(args)))
        n = int(rows.value)
        kv = self.dev.alloc(2 * num_heads * n * 128 * 2, L.DTYPE_BF16)
        L.check(self.lib.relux_cuda_memset(self.dev.h, kv.ptr, 0xFF, kv.nbytes))   # NaN bit patterns: a row the kernel misses shows
        base = self.dev.alloc((n_seqs + 1) * 4, L.DTYPE_F32)
        args.kv_out, args.seq_base, args.rows_total = kv.ptr, base.ptr, n
        L.check(self.lib.relux_mla_expand_kv(self.h, C.byref(args)))
        out = kv.download((2, num_heads, n, 128), np.uint16)
        sb = base.download((n_seqs + 1,), np.int32)
        kv.free(); base.free()
        return out[0], out[1], sb

    def selftest_wait(self, polls):
        """Runs the bounded-wait self test (a wait nobody answers, `polls` polls): afterwards status() reports ERR_TIMEOUT."""
        L.check(self.lib.relux_pool_selftest_wait(self.h, int(polls)))

    def kernel_ms_list(self, last_n):
        """Device times (ms) of the attention kernel of the most recent `last_n` decode / verify calls, oldest first."""
        out = np.zeros(int(last_n), np.float32)
        n = C.c_int32()
        L.check(self.lib.relux_pool_kernel_ms_list(self.h, int(last_n), out.ctypes.data, C.byref(n)))
        return out[:n.value]

    def _append_args(self, layer, a, b, n_seqs, seq_ids, n_new, layout, advance, dtype, pipelined=False):
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        nn = None if n_new is None else np.ascontiguousarray(n_new, dtype=np.int32)
        self._keep = [ids, nn, a, b]
        return L.AppendArgs(layer=layer, n_seqs=n_seqs, seq_ids=_ptr(ids), n_new=_ptr(nn), a=_ptr(a), b=_ptr(b),
                            dtype=_dtype_flag(a, dtype), mem=_mem(a), layout=layout, advance=int(advance),
                            flags=L.CALL_PIPELINED if pipelined else 0)

    def append(self, layer, a, b, n_seqs, seq_ids=None, n_new=None, layout=L.LAYOUT_TOKEN_MAJOR, advance=True, dtype=None,
               pipelined=False):
        """MLA: a = c_kv [rows, dC], b = k_rope [rows, dHR].  GQA: a = K, b = V.  pipelined: host inputs travel on the copy
        stream and the call returns once queued (see RELUX_CALL_PIPELINED in include/relux_cuda.h)."""
        args = self._append_args(layer, a, b, n_seqs, seq_ids, n_new, layout, advance, dtype, pipelined)
        fn = self.lib.relux_mla_append if self.kind == L.POOL_MLA else self.lib.relux_gqa_append
        L.check(fn(self.h, C.byref(args)))

    def _attn_args(self, layer, n_seqs, q, q_rope, out, num_heads, head_dim, scale, q_tokens, extra_tokens, causal, mode,
                   w_uk, w_uv, seq_ids, q_layout, out_layout, q_dtype, out_dtype, pipelined=False):
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        self._keep2 = [ids, q, q_rope, out]
        return L.AttnArgs(layer=layer, n_seqs=n_seqs, seq_ids=_ptr(ids), q_tokens=q_tokens, extra_tokens=extra_tokens,
                          causal=int(causal), num_heads=num_heads, head_dim=head_dim, scale=scale, q=_ptr(q), q_rope=_ptr(q_rope),
                          q_dtype=_dtype_flag(q, q_dtype), q_mem=_mem(q), q_layout=q_layout, w_uk=_ptr(w_uk), w_uv=_ptr(w_uv),
                          out=_ptr(out), out_dtype=_dtype_flag(out, out_dtype), out_mem=_mem(out), out_layout=out_layout, mode=mode,
                          flags=L.CALL_PIPELINED if pipelined else 0)

    def decode(self, layer, n_seqs, q, out, num_heads, head_dim, scale, q_rope=None, w_uk=None, w_uv=None, q_tokens=1,
               extra_tokens=0, causal=True, mode=L.ATTN_FAST, seq_ids=None, q_layout=L.LAYOUT_TOKEN_MAJOR,
               out_layout=L.LAYOUT_TOKEN_MAJOR, q_dtype=None, out_dtype=None, pipelined=False):
        args = self._attn_args(layer, n_seqs, q, q_rope, out, num_heads, head_dim, scale, q_tokens, extra_tokens, causal, mode,
                               w_uk, w_uv, seq_ids, q_layout, out_layout, q_dtype, out_dtype, pipelined)
        fn = self.lib.relux_mla_decode if self.kind == L.POOL_MLA else self.lib.relux_gqa_decode
        L.check(fn(self.h, C.byref(args)))

    def decode_noalloc(self, layer, n_seqs, q, out, num_heads, head_dim, scale, q_tokens=1, extra_tokens=0, causal=True,
                       seq_ids=None):
        """GQA decode through the entry point that allocates no device memory (fixed 16 MiB scratch, device-resident
        q and f32 out only; see relux_gqa_decode_noalloc in include/relux_cuda.h)."""
        args = self._attn_args(layer, n_seqs, q, None, out, num_heads, head_dim, scale, q_tokens, extra_tokens, causal, L.ATTN_FAST,
                               None, None, seq_ids, L.LAYOUT_TOKEN_MAJOR, L.LAYOUT_TOKEN_MAJOR, None, None)
        L.check(self.lib.relux_gqa_decode_noalloc(self.h, C.byref(args)))

    def verify(self, layer, n_seqs, q, out, draft_a, draft_b, num_heads, head_dim, scale, q_tokens, q_rope=None, w_uk=None,
               w_uv=None, mode=L.ATTN_FAST, seq_ids=None, kv_layout=L.LAYOUT_TOKEN_MAJOR, q_dtype=None, out_dtype=None,
               kv_dtype=None, pipelined=False):
        """Speculative verify: draft rows are written past the cursor, q_tokens rows attend causally."""
        n_new = np.full(n_seqs, q_tokens, np.int32)
        ap = self._append_args(layer, draft_a, draft_b, n_seqs, seq_ids, n_new, kv_layout, False, kv_dtype, pipelined)
        at = self._attn_args(layer, n_seqs, q, q_rope, out, num_heads, head_dim, scale, q_tokens, q_tokens, True, mode, w_uk, w_uv,
                             seq_ids, L.LAYOUT_TOKEN_MAJOR, L.LAYOUT_TOKEN_MAJOR, q_dtype, out_dtype, pipelined)
        fn = self.lib.relux_mla_verify if self.kind == L.POOL_MLA else self.lib.relux_gqa_verify
        L.check(fn(self.h, C.byref(at), C.byref(ap)))

    def step(self, layer, n_seqs, new_a, new_b, q, out, num_heads, head_dim, scale, q_rope=None, w_uk=None, w_uv=None, n_new=None,
             mode=L.ATTN_FAST, seq_ids=None, kv_layout=L.LAYOUT_TOKEN_MAJOR, q_dtype=None, out_dtype=None, kv_dtype=None, pipelined=False):
        """One decode step in one call: append the new rows, then attend (relux_mla_step / relux_gqa_step)."""
        ap = self._append_args(layer, new_a, new_b, n_seqs, seq_ids, n_new, kv_layout, True, kv_dtype, pipelined)
        at = self._attn_args(layer, n_seqs, q, q_rope, out, num_heads, head_dim, scale, 1, 0, True, mode, w_uk, w_uv, seq_ids,
                             L.LAYOUT_TOKEN_MAJOR, L.LAYOUT_TOKEN_MAJOR, q_dtype, out_dtype, pipelined)
        fn = self.lib.relux_mla_step if self.kind == L.POOL_MLA else self.lib.relux_gqa_step
        L.check(fn(self.h, C.byref(ap), C.byref(at)))

    def spec_accept(self, n_seqs, k, vocab, draft_tokens, draft_logits, target_logits, draws, temperature=1.0, top_k=0,
                    top_p=1.0, min_p=0.0, mode=L.ATTN_FAST, commit=False, seq_ids=None):
        """acceptPhase + resampleRejected (speculative.go:211-295) for n_seqs sequences, ending in Sampler.Sample
        (sampler.go:73-218) when all k draft tokens pass.  The four inputs are all numpy arrays or all device buffers;
        draws [n_seqs, k + 1] are the uniform numbers the reference would take from its generator.  k = 0 samples one
        token per row of target_logits [n_seqs, vocab].  Returns (n_accepted, next_token) as int32 arrays.
        commit=True grows every layer of each sequence by n_accepted + 1 rows (the rows a verify call left past the cursor)."""
        mems = {_mem(a) for a in (draft_tokens, draft_logits, target_logits, draws) if a is not None}
        if len(mems) != 1:
            raise TypeError("spec_accept: inputs must be all host arrays or all device buffers")
        keep = []

        def host(a, dt):
            if a is None or _mem(a) == L.MEM_DEVICE:
                return a
            a = np.ascontiguousarray(a, dtype=dt)
            keep.append(a)
            return a

        draft_tokens, draft_logits = host(draft_tokens, np.int32), host(draft_logits, np.float32)
        target_logits, draws = host(target_logits, np.float32), host(draws, np.float32)
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        n_acc = np.full(n_seqs, -1, np.int32)
        nxt = np.full(n_seqs, -1, np.int32)
        args = L.SpecAcceptArgs(n_seqs=n_seqs, k=k, vocab=vocab, mem=mems.pop(), draft_tokens=_ptr(draft_tokens),
                                draft_logits=_ptr(draft_logits), target_logits=_ptr(target_logits), draws=_ptr(draws),
                                sampler=L.SamplerParams(float(temperature), int(top_k), float(top_p), float(min_p)), mode=mode,
                                commit=int(commit), seq_ids=_ptr(ids), n_accepted=n_acc.ctypes.data, next_token=nxt.ctypes.data)
        L.check(self.lib.relux_spec_accept(self.h, C.byref(args)))
        return n_acc, nxt

    def sample(self, logits, draws, vocab=None, n_rows=None, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, mode=L.ATTN_FAST,
               prev_tokens=None, repeat_penalty=1.0, frequency_penalty=0.0, presence_penalty=0.0, repeat_window=0):
        """Sampler.Sample (sampler.go:73-218) for a batch of rows: logits [n, vocab] and draws [n] as numpy arrays or
        device buffers (then pass n_rows and vocab); prev_tokens: one sequence of earlier token ids per row for the
        repetition penalties (sampler.go:221-266), or None.  Returns the token ids (int32 array)."""
        if n_rows is None:
            n_rows, vocab = logits.shape
        if _mem(logits) != _mem(draws):
            raise TypeError("sample: logits and draws must both be host arrays or both device buffers")
        if _mem(logits) == L.MEM_HOST:
            logits = np.ascontiguousarray(logits, dtype=np.float32)
            draws = np.ascontiguousarray(draws, dtype=np.float32)
        prev = plen = None
        stride = 0
        if prev_tokens is not None:
            plen = np.asarray([len(t) for t in prev_tokens], np.int32)
            stride = int(max(1, plen.max() if plen.size else 1))
            prev = np.zeros((n_rows, stride), np.int32)
            for i, t in enumerate(prev_tokens):
                prev[i, :len(t)] = np.asarray(t, np.int32)
        toks = np.full(n_rows, -1, np.int32)
        args = L.SampleArgs(n_rows=n_rows, vocab=vocab, mem=_mem(logits), mode=mode, logits=_ptr(logits), draws=_ptr(draws),
                            sampler=L.SamplerParams(float(temperature), int(top_k), float(top_p), float(min_p)),
                            repeat_penalty=float(repeat_penalty), frequency_penalty=float(frequency_penalty),
                            presence_penalty=float(presence_penalty), repeat_window=int(repeat_window), prev_tokens=_ptr(prev),
                            prev_len=_ptr(plen), prev_stride=stride, tokens=toks.ctypes.data)
        L.check(self.lib.relux_sampler_sample(self.h, C.byref(args)))
        return toks

    def forward_cached(self, layer, n_seqs, x, out, weights, d_model, num_heads, q_tokens=1, causal=True, rope_base=0.0,
                       mode=L.ATTN_FAST, seq_ids=None, rope=True, advance=True):
        if self.kind == L.POOL_GQA:
            return self._gqa_forward_cached(layer, n_seqs, x, out, weights, d_model, num_heads, q_tokens, causal, rope_base, mode,
                                            seq_ids, rope, advance)
        return self._mla_forward_cached(layer, n_seqs, x, out, weights, d_model, num_heads, q_tokens, causal, rope_base, mode, seq_ids)

    def _gqa_forward_cached(self, layer, n_seqs, x, out, weights, d_model, num_heads, q_tokens, causal, rope_base, mode, seq_ids,
                            rope, advance):
        """One GQA layer step (MHA.forwardCached, mha.go:245-369): x [n_seqs, q_tokens, d_model] float32 -> out of the
        same shape; `weights` maps w_q, w_k, w_v, w_o to device buffers of bf16 bits in the reference's [in, out] layout.
        advance=False leaves the q_tokens new rows past the cursor (speculative verify)."""
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        w = L.GqaLayerWeights(**{k: _ptr(weights[k]) for k in ("w_q", "w_k", "w_v", "w_o")})
        args = L.GqaLayerArgs(layer=layer, n_seqs=n_seqs, seq_ids=_ptr(ids), q_tokens=q_tokens, causal=int(causal), d_model=d_model,
                              num_heads=num_heads, rope=int(rope), rope_base=float(rope_base), advance=int(advance), mode=mode,
                              x=_ptr(x), x_dtype=_dtype_flag(x), x_mem=_mem(x), out=_ptr(out), out_mem=_mem(out), w=C.pointer(w))
        L.check(self.lib.relux_gqa_forward_cached(self.h, C.byref(args)))

    def _mla_forward_cached(self, layer, n_seqs, x, out, weights, d_model, num_heads, q_tokens=1, causal=True, rope_base=0.0,
                            mode=L.ATTN_FAST, seq_ids=None):
        """One MLA layer step (MLA.forwardCached, mla.go:272-397): x [n_seqs, q_tokens, d_model] float32 ->
        out [n_seqs, q_tokens, d_model] float32; `weights` maps w_q, w_qr, w_dkv, w_kr, w_uk, w_uv, w_o to device
        buffers of bf16 bits in the reference's [in, out] layout.  Appends q_tokens rows per sequence."""
        ids = None if seq_ids is None else np.ascontiguousarray(seq_ids, dtype=np.int32)
        w = L.MlaLayerWeights(**{k: _ptr(weights[k]) for k in ("w_q", "w_qr", "w_dkv", "w_kr", "w_uk", "w_uv", "w_o")})
        args = L.MlaLayerArgs(layer=layer, n_seqs=n_seqs, seq_ids=_ptr(ids), q_tokens=q_tokens, causal=int(causal), d_model=d_model,
                              num_heads=num_heads, rope_base=float(rope_base), mode=mode, x=_ptr(x), x_dtype=_dtype_flag(x),
                              x_mem=_mem(x), out=_ptr(out), out_mem=_mem(out), w=C.pointer(w))
        L.check(self.lib.relux_mla_forward_cached(self.h, C.byref(args)))

    def last_kernel_ms(self):
        ms = C.c_float()
        L.check(self.lib.relux_pool_last_kernel_ms(self.h, C.byref(ms)))
        return ms.value

    def save_file(self, seq, path, max_len):
        """Writes sequence `seq` in the layout of the reference's NewKVCacheFile / NewMLACacheFile."""
        L.check(self.lib.relux_seq_save_file(self.h, int(seq), os.fsencode(path), int(max_len)))

    def load_file(self, seq, path, max_len, layer_len):
        """Resets sequence `seq` and fills it from such a file; layer_len[l] rows are taken for layer l."""
        ll = np.ascontiguousarray(layer_len, dtype=np.int32)
        L.check(self.lib.relux_seq_load_file(self.h, int(seq), os.fsencode(path), int(max_len), ll.ctypes.data))

    def mean_projection_ms(self, last_n):
        """(mean device time of the input-projection GEMM over the last `last_n` forward_cached calls, calls counted)."""
        ms, n = C.c_float(), C.c_int32()
        L.check(self.lib.relux_pool_projection_ms_mean(self.h, int(last_n), C.byref(ms), C.byref(n)))
        return ms.value, n.value

    def mean_kernel_ms(self, last_n):
        """(mean device time of the attention kernel over the last `last_n` decode / verify calls, calls counted)."""
        ms, n = C.c_float(), C.c_int32()
        L.check(self.lib.relux_pool_kernel_ms_mean(self.h, int(last_n), C.byref(ms), C.byref(n)))
        return ms.value, n.value


BFloat16 = "bf16"


class KVCache:
    """NewKVCacheSized(numLayers, maxLen, numKVHeads, headDim, BFloat16)   kvcache.go:66-93.
    One sequence, every layer; tensors follow the reference's shapes: K/V [1, numKVHeads, newLen, headDim]."""

    def __init__(self, dev, num_layers, max_len, num_kv_heads, head_dim, page_tokens=64, reference_compat=False):
        if num_layers <= 0:
            raise ValueError("NewKVCacheSized: numLayers=%d, must be > 0" % num_layers)
        if max_len <= 0:
            raise ValueError("NewKVCacheSized: maxLen=%d, must be > 0" % max_len)
        pages = (max_len + page_tokens - 1) // page_tokens
        self.pool = Pool(dev, L.POOL_GQA, num_layers, pages, page_tokens, 1, pages, num_kv_heads=num_kv_heads, head_dim=head_dim,
                         reference_compat=reference_compat)
        self.seq = self.pool.seq_alloc(max_len)
        self.num_layers, self.max_len, self.num_kv_heads, self.head_dim = num_layers, max_len, num_kv_heads, head_dim

    def DType(self):
        return BFloat16

    def TotalLen(self, layer):
        return self.pool.seq_len(layer, self.seq)

    def Append(self, layer, new_k, new_v):
        if not (0 <= layer < self.num_layers):
            raise IndexError("KVCache.Append: layerIdx=%d out of range [0, %d)" % (layer, self.num_layers))
        new_k = np.ascontiguousarray(new_k, dtype=np.float32)
        new_v = np.ascontiguousarray(new_v, dtype=np.float32)
        if new_k.shape != new_v.shape:
            raise ValueError("KVCache.Append: K and V shape mismatch: %s vs %s" % (new_k.shape, new_v.shape))
        if new_k.ndim < 3:
            raise ValueError("KVCache.Append: K rank=%d, want >= 3 [batch, heads, seq, headDim]" % new_k.ndim)
        n_new = new_k.shape[-2]
        try:
            self.pool.append(layer, new_k, new_v, 1, seq_ids=[self.seq], n_new=[n_new], layout=L.LAYOUT_HEAD_MAJOR)
        except L.ReluxCudaError as e:
            if e.code == L.ERR_OVERFLOW:
                raise OverflowError(str(e))
            raise

    def View(self, layer):
        """Returns (K, V) as bf16 bit patterns shaped [1, numKVHeads, total, headDim], or (None, None)."""
        if not (0 <= layer < self.num_layers):
            raise IndexError("KVCache.View: layerIdx=%d out of range" % layer)
        t = self.TotalLen(layer)
        if t == 0:
            return None, None
        k, v = self.pool.read_rows(layer, self.seq, 0, t)  # [t, Hkv, D]
        return (np.ascontiguousarray(k.transpose(1, 0, 2))[None], np.ascontiguousarray(v.transpose(1, 0, 2))[None])

    def Reset(self):
        self.pool.set_len(-1, [0], [self.seq])

    def attend(self, layer, q, scale, causal=True, mode=L.ATTN_FAST, extra_tokens=0):
        """q [1, H, S, D] float32 (post-RoPE) -> attention output [1, H, S, D] float32 over the cached rows;
        the S query rows are the last S cached rows (append first, then attend: mha.go:287-296)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        _, H, S, D = q.shape
        out = np.empty_like(q)
        self.pool.decode(layer, 1, q, out, H, D, scale, q_tokens=S, extra_tokens=extra_tokens, causal=causal, mode=mode,
                         seq_ids=[self.seq], q_layout=L.LAYOUT_HEAD_MAJOR, out_layout=L.LAYOUT_HEAD_MAJOR)
        return out

    def close(self):
        self.pool.destroy()


class MLACache:
    """NewMLACache(numLayers, maxLen, dC, dHR)   mla_cache.go:38-59 (rows are stored as bf16 here)."""

    def __init__(self, dev, num_layers, max_len, dC, dHR, page_tokens=64, reference_compat=False):
        if num_layers <= 0:
            raise ValueError("NewMLACache: numLayers=%d, must be > 0" % num_layers)
        if max_len <= 0:
            raise ValueError("NewMLACache: maxLen=%d, must be > 0" % max_len)
        pages = (max_len + page_tokens - 1) // page_tokens
        self.pool = Pool(dev, L.POOL_MLA, num_layers, pages, page_tokens, 1, pages, dC=dC, dHR=dHR, reference_compat=reference_compat)
        self.seq = self.pool.seq_alloc(max_len)
        self.num_layers, self.max_len, self.dC, self.dHR = num_layers, max_len, dC, dHR

    def TotalLen(self, layer):
        return self.pool.seq_len(layer, self.seq)

    def Append(self, layer, new_c, new_kr):
        if not (0 <= layer < self.num_layers):
            raise IndexError("MLACache.Append: layerIdx=%d out of range [0, %d)" % (layer, self.num_layers))
        c = np.ascontiguousarray(new_c, dtype=np.float32)
        r = np.ascontiguousarray(new_kr, dtype=np.float32)
        n_new = c.shape[-2]
        try:
            self.pool.append(layer, c, r, 1, seq_ids=[self.seq], n_new=[n_new])
        except L.ReluxCudaError as e:
            if e.code == L.ERR_OVERFLOW:
                raise OverflowError(str(e))
            raise

    def View(self, layer):
        if not (0 <= layer < self.num_layers):
            raise IndexError("MLACache.View: layerIdx=%d out of range" % layer)
        t = self.TotalLen(layer)
        if t == 0:
            return None, None
        c, r = self.pool.read_rows(layer, self.seq, 0, t)
        return c[None], r[None]

    def Reset(self):
        self.pool.set_len(-1, [0], [self.seq])

    def attend(self, layer, qc, qr, w_uk, w_uv, scale, causal=True, mode=L.ATTN_FAST, extra_tokens=0):
        """qc [1,H,S,Dh], qr [1,H,S,dHR] float32; w_uk / w_uv device buffers [dC, H*Dh] bf16 -> [1,H,S,Dh] float32."""
        qc = np.ascontiguousarray(qc, dtype=np.float32)
        qr = np.ascontiguousarray(qr, dtype=np.float32)
        _, H, S, Dh = qc.shape
        out = np.empty_like(qc)
        self.pool.decode(layer, 1, qc, out, H, Dh, scale, q_rope=qr, w_uk=w_uk, w_uv=w_uv, q_tokens=S, extra_tokens=extra_tokens,
                         causal=causal, mode=mode, seq_ids=[self.seq], q_layout=L.LAYOUT_HEAD_MAJOR, out_layout=L.LAYOUT_HEAD_MAJOR)
        return out

    def close(self):
        self.pool.destroy()
