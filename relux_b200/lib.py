"""ctypes binding of librelux_cuda.so (the C ABI declared in include/relux_cuda.h).

This is the Python stand-in for the purego binding a Go caller would write: same entry points, same
argument structs.  There is no fallback: if the shared library is missing or a call fails, an exception
is raised.
"""
import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "librelux_cuda.so")
CSRC = os.path.join(_HERE, "csrc")

OK = 0
ERR_INVALID_ARG, ERR_CUDA, ERR_OUT_OF_MEMORY, ERR_POOL_EXHAUSTED, ERR_OVERFLOW = -1, -2, -3, -4, -5
ERR_BAD_PAGE, ERR_TIMEOUT, ERR_BAD_HANDLE, ERR_UNSUPPORTED, ERR_NO_DEVICE = -6, -7, -8, -9, -10
DTYPE_F32, DTYPE_BF16 = 0, 1
MEM_HOST, MEM_DEVICE = 0, 1
LAYOUT_TOKEN_MAJOR, LAYOUT_HEAD_MAJOR = 0, 1
POOL_MLA, POOL_GQA = 0, 1
ATTN_FAST, ATTN_REFERENCE, ATTN_REFERENCE_FAITHFUL = 0, 1, 2
POOL_FLAG_REFERENCE_COMPAT = 1
CALL_PIPELINED = 1
(TUNE_MLA_GENERIC, TUNE_MLA_WORKERS, TUNE_CHUNK_PAGES, TUNE_GEMM_GENERIC, TUNE_GEMM_SPLIT, TUNE_GQA_PROMPT_PARTIAL_MB, TUNE_SEL_CLUSTER,
 TUNE_SEL_LOOKAHEAD, TUNE_SEL_BATCHED, TUNE_GQA_PROMPT_SLICES, TUNE_MLA_PROMPT_MIN_TOKENS, TUNE_MLA_PROMPT_SCRATCH_MB,
 TUNE_KERNEL_TIMING_STRIDE, TUNE_CHAINED_LAUNCHES) = range(14)

# Every symbol include/relux_cuda.h declares; tests check that the library exports each one.
EXPORTS = [
    "relux_cuda_version", "relux_cuda_device_count", "relux_cuda_device_open", "relux_cuda_device_close", "relux_cuda_sync",
    "relux_cuda_last_error", "relux_cuda_device_info", "relux_cuda_launch_count", "relux_cuda_stream", "relux_cuda_dev_alloc",
    "relux_cuda_dev_free", "relux_cuda_host_alloc", "relux_cuda_host_free", "relux_cuda_h2d", "relux_cuda_d2h",
    "relux_cuda_memset", "relux_cuda_event_create", "relux_cuda_event_record", "relux_cuda_event_elapsed_ms",
    "relux_cuda_event_destroy", "relux_cuda_flush_l2", "relux_pool_create", "relux_pool_destroy", "relux_pool_reset",
    "relux_pool_set_tables", "relux_seq_alloc", "relux_seq_free", "relux_seq_extend", "relux_seq_len", "relux_seq_set_len", "relux_pool_status",
    "relux_pool_read_rows", "relux_mla_append", "relux_gqa_append", "relux_mla_decode", "relux_gqa_decode", "relux_gqa_verify",
    "relux_mla_verify", "relux_pool_last_kernel_ms", "relux_pool_kernel_ms_mean", "relux_mla_forward_cached", "relux_gqa_forward_cached", "relux_stream_partition", "relux_seq_save_file", "relux_seq_load_file", "relux_pool_projection_ms_mean", "relux_gqa_decode_noalloc",
    "relux_spec_accept", "relux_sampler_sample", "relux_pool_tune", "relux_pool_kernel_ms_list", "relux_matmul_f32_bf16",
    "relux_mla_import_weights", "relux_pool_selftest_wait", "relux_pool_wait_output", "relux_mla_step", "relux_gqa_step", "relux_mla_expand_kv",
]


class PoolParams(C.Structure):
    _fields_ = [("kind", C.c_int32), ("num_layers", C.c_int32), ("num_pages", C.c_int32), ("page_tokens", C.c_int32),
                ("max_seqs", C.c_int32), ("max_pages_per_seq", C.c_int32), ("mla_dc", C.c_int32), ("mla_dhr", C.c_int32),
                ("gqa_num_kv_heads", C.c_int32), ("gqa_head_dim", C.c_int32), ("flags", C.c_int32), ("reserved", C.c_int32 * 5)]


class ReadRowsArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("seq_id", C.c_int32), ("tok0", C.c_int32), ("n_tokens", C.c_int32), ("dst_a", C.c_void_p),
                ("dst_b", C.c_void_p), ("reserved", C.c_int32 * 4)]


class StreamPartitionArgs(C.Structure):
    _fields_ = [("pages", C.c_void_p), ("n_seqs", C.c_int32), ("workers", C.c_int32), ("page_multiple", C.c_int32), ("cap", C.c_int32),
                ("range_pages_out", C.c_void_p), ("workers_out", C.c_void_p), ("items_out", C.c_void_p), ("worker_first", C.c_void_p),
                ("chunk_off", C.c_void_p)]


class MatmulArgs(C.Structure):
    _fields_ = [("m", C.c_int32), ("k", C.c_int32), ("n", C.c_int32), ("mode", C.c_int32), ("a", C.c_void_p), ("a_mem", C.c_int32),
                ("c_mem", C.c_int32), ("b", C.c_void_p), ("c", C.c_void_p), ("reserved", C.c_int32 * 4)]


class AppendArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("n_seqs", C.c_int32), ("seq_ids", C.c_void_p), ("n_new", C.c_void_p),
                ("a", C.c_void_p), ("b", C.c_void_p), ("dtype", C.c_int32), ("mem", C.c_int32), ("layout", C.c_int32),
                ("advance", C.c_int32), ("flags", C.c_int32), ("reserved", C.c_int32 * 3)]


class AttnArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("n_seqs", C.c_int32), ("seq_ids", C.c_void_p), ("q_tokens", C.c_int32),
                ("extra_tokens", C.c_int32), ("causal", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
                ("scale", C.c_float), ("q", C.c_void_p), ("q_rope", C.c_void_p), ("q_dtype", C.c_int32), ("q_mem", C.c_int32),
                ("q_layout", C.c_int32), ("w_uk", C.c_void_p), ("w_uv", C.c_void_p), ("out", C.c_void_p),
                ("out_dtype", C.c_int32), ("out_mem", C.c_int32), ("out_layout", C.c_int32), ("mode", C.c_int32),
                ("flags", C.c_int32), ("reserved", C.c_int32 * 4)]


class MlaLayerWeights(C.Structure):
    _fields_ = [("w_q", C.c_void_p), ("w_qr", C.c_void_p), ("w_dkv", C.c_void_p), ("w_kr", C.c_void_p), ("w_uk", C.c_void_p),
                ("w_uv", C.c_void_p), ("w_o", C.c_void_p)]


class MlaLayerArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("n_seqs", C.c_int32), ("seq_ids", C.c_void_p), ("q_tokens", C.c_int32),
                ("causal", C.c_int32), ("d_model", C.c_int32), ("num_heads", C.c_int32), ("rope_base", C.c_float),
                ("mode", C.c_int32), ("x", C.c_void_p), ("x_dtype", C.c_int32), ("x_mem", C.c_int32), ("out", C.c_void_p),
                ("out_mem", C.c_int32), ("reserved", C.c_int32 * 3), ("w", C.POINTER(MlaLayerWeights))]


class MlaImportArgs(C.Structure):
    _fields_ = [("d_model", C.c_int32), ("num_heads", C.c_int32), ("nope_dim", C.c_int32), ("rope_dim", C.c_int32), ("v_dim", C.c_int32),
                ("dc", C.c_int32), ("src_dtype", C.c_int32), ("src_mem", C.c_int32), ("fused_rope", C.c_int32),
                ("reserved", C.c_int32 * 3), ("q_proj", C.c_void_p), ("kv_a_proj_with_mqa", C.c_void_p), ("kv_b_proj", C.c_void_p),
                ("o_proj", C.c_void_p), ("q_pe_proj", C.c_void_p), ("k_pe_proj", C.c_void_p), ("dst", C.POINTER(MlaLayerWeights))]


class MlaExpandArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("n_seqs", C.c_int32), ("seq_ids", C.c_void_p), ("extra_tokens", C.c_int32), ("num_heads", C.c_int32),
                ("w_uk", C.c_void_p), ("w_uv", C.c_void_p), ("kv_out", C.c_void_p), ("seq_base", C.c_void_p), ("rows_total", C.c_int64),
                ("rows_total_out", C.POINTER(C.c_int64)), ("reserved", C.c_int32 * 4)]


class GqaLayerWeights(C.Structure):
    _fields_ = [("w_q", C.c_void_p), ("w_k", C.c_void_p), ("w_v", C.c_void_p), ("w_o", C.c_void_p)]


class GqaLayerArgs(C.Structure):
    _fields_ = [("layer", C.c_int32), ("n_seqs", C.c_int32), ("seq_ids", C.c_void_p), ("q_tokens", C.c_int32),
                ("causal", C.c_int32), ("d_model", C.c_int32), ("num_heads", C.c_int32), ("rope", C.c_int32),
                ("rope_base", C.c_float), ("advance", C.c_int32), ("mode", C.c_int32), ("x", C.c_void_p), ("x_dtype", C.c_int32),
                ("x_mem", C.c_int32), ("out", C.c_void_p), ("out_mem", C.c_int32), ("reserved", C.c_int32 * 3),
                ("w", C.POINTER(GqaLayerWeights))]


class SamplerParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("min_p", C.c_float)]


class SpecAcceptArgs(C.Structure):
    _fields_ = [("n_seqs", C.c_int32), ("k", C.c_int32), ("vocab", C.c_int32), ("mem", C.c_int32),
                ("draft_tokens", C.c_void_p), ("draft_logits", C.c_void_p), ("target_logits", C.c_void_p),
                ("draws", C.c_void_p), ("sampler", SamplerParams), ("mode", C.c_int32), ("commit", C.c_int32),
                ("seq_ids", C.c_void_p), ("n_accepted", C.c_void_p), ("next_token", C.c_void_p), ("reserved", C.c_int32 * 4)]


class SampleArgs(C.Structure):
    _fields_ = [("n_rows", C.c_int32), ("vocab", C.c_int32), ("mem", C.c_int32), ("mode", C.c_int32), ("logits", C.c_void_p),
                ("draws", C.c_void_p), ("sampler", SamplerParams), ("repeat_penalty", C.c_float), ("frequency_penalty", C.c_float),
                ("presence_penalty", C.c_float), ("repeat_window", C.c_int32), ("prev_tokens", C.c_void_p), ("prev_len", C.c_void_p),
                ("prev_stride", C.c_int32), ("reserved", C.c_int32 * 3), ("tokens", C.c_void_p)]


class ReluxCudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("librelux_cuda status %d: %s" % (code, msg))
        self.code = code


def build(force=False, verbose=False):
    """Compiles librelux_cuda.so for sm_100a with nvcc (cross-compiles without a GPU)."""
    args = ["make", "-C", CSRC, "-j8"] + ([] if verbose else ["-s"])
    if force:
        subprocess.check_call(["make", "-C", CSRC, "clean", "-s"])
    subprocess.check_call(args)
    return SO_PATH


_lib = None


def load():
    """Loads the shared library (never builds, never falls back)."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise FileNotFoundError("%s is missing: run `python -c 'import __graft_entry__ as g; g.build()'` or "
                                    "`make -C relux_b200/csrc`; there is no CPU fallback" % SO_PATH)
        L = C.CDLL(SO_PATH)
        for name in EXPORTS:
            getattr(L, name).restype = C.c_int32
        L.relux_cuda_dev_alloc.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]
        L.relux_cuda_host_alloc.argtypes = [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]
        L.relux_cuda_dev_free.argtypes = [C.c_void_p, C.c_void_p]
        L.relux_cuda_host_free.argtypes = [C.c_void_p, C.c_void_p]
        L.relux_cuda_h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.relux_cuda_d2h.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.relux_cuda_memset.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_size_t]
        L.relux_cuda_sync.argtypes = [C.c_void_p]
        L.relux_cuda_device_close.argtypes = [C.c_void_p]
        L.relux_cuda_flush_l2.argtypes = [C.c_void_p]
        L.relux_cuda_event_create.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        L.relux_cuda_event_record.argtypes = [C.c_void_p, C.c_void_p]
        L.relux_cuda_event_elapsed_ms.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
        L.relux_cuda_event_destroy.argtypes = [C.c_void_p, C.c_void_p]
        L.relux_pool_create.argtypes = [C.c_void_p, C.POINTER(PoolParams), C.POINTER(C.c_void_p)]
        for n in ("relux_pool_destroy", "relux_pool_reset"):
            getattr(L, n).argtypes = [C.c_void_p]
        L.relux_pool_set_tables.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        L.relux_seq_alloc.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_int32)]
        L.relux_seq_free.argtypes = [C.c_void_p, C.c_int32]
        L.relux_seq_extend.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        L.relux_seq_len.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]
        L.relux_seq_set_len.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]
        L.relux_pool_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
        L.relux_pool_read_rows.argtypes = [C.c_void_p, C.POINTER(ReadRowsArgs)]
        L.relux_pool_tune.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        L.relux_pool_wait_output.argtypes = [C.c_void_p, C.c_int32]
        L.relux_pool_kernel_ms_list.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.POINTER(C.c_int32)]
        L.relux_matmul_f32_bf16.argtypes = [C.c_void_p, C.POINTER(MatmulArgs)]
        L.relux_mla_import_weights.argtypes = [C.c_void_p, C.POINTER(MlaImportArgs)]
        L.relux_mla_expand_kv.argtypes = [C.c_void_p, C.POINTER(MlaExpandArgs)]
        L.relux_pool_selftest_wait.argtypes = [C.c_void_p, C.c_int32]
        for n in ("relux_mla_append", "relux_gqa_append"):
            getattr(L, n).argtypes = [C.c_void_p, C.POINTER(AppendArgs)]
        for n in ("relux_mla_decode", "relux_gqa_decode", "relux_gqa_decode_noalloc"):
            getattr(L, n).argtypes = [C.c_void_p, C.POINTER(AttnArgs)]
        for n in ("relux_gqa_verify", "relux_mla_verify"):
            getattr(L, n).argtypes = [C.c_void_p, C.POINTER(AttnArgs), C.POINTER(AppendArgs)]
        for n in ("relux_gqa_step", "relux_mla_step"):
            getattr(L, n).argtypes = [C.c_void_p, C.POINTER(AppendArgs), C.POINTER(AttnArgs)]
        L.relux_pool_projection_ms_mean.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int32)]
        L.relux_stream_partition.argtypes = [C.POINTER(StreamPartitionArgs)]
        L.relux_seq_save_file.argtypes = [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32]
        L.relux_seq_load_file.argtypes = [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32, C.c_void_p]
        L.relux_gqa_forward_cached.argtypes = [C.c_void_p, C.POINTER(GqaLayerArgs)]
        L.relux_mla_forward_cached.argtypes = [C.c_void_p, C.POINTER(MlaLayerArgs)]
        L.relux_spec_accept.argtypes = [C.c_void_p, C.POINTER(SpecAcceptArgs)]
        L.relux_sampler_sample.argtypes = [C.c_void_p, C.POINTER(SampleArgs)]
        L.relux_pool_last_kernel_ms.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
        L.relux_pool_kernel_ms_mean.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int32)]
        L.relux_cuda_launch_count.argtypes = [C.c_void_p, C.POINTER(C.c_int64)]
        L.relux_cuda_stream.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        _lib = L
    return _lib


def last_error():
    buf = C.create_string_buffer(512)
    load().relux_cuda_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc):
    if rc != OK:
        raise ReluxCudaError(rc, last_error())
