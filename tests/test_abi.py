"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the header declares,
and fails cleanly (status + message, no crash) when no GPU is present."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def so():
    import __graft_entry__ as g
    g.build()
    from relux_b200 import lib as L
    return L


def header_functions():
    src = open(os.path.join(ROOT, "include", "relux_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\bint32_t\s+(relux_\w+)\s*\(", src)))


def test_header_and_binding_agree(so):
    assert header_functions() == sorted(so.EXPORTS)


def test_every_declared_symbol_is_exported(so):
    lib = C.CDLL(so.SO_PATH)
    for name in header_functions():
        assert hasattr(lib, name), "librelux_cuda.so does not export %s" % name


def test_version_and_error_text(so):
    lib = so.load()
    assert lib.relux_cuda_version() == 1
    buf = C.create_string_buffer(64)
    assert lib.relux_cuda_last_error(buf, 64) == 0


def test_bad_handles_are_rejected(so):
    lib = so.load()
    assert lib.relux_cuda_sync(None) == so.ERR_BAD_HANDLE
    assert lib.relux_pool_destroy(None) == so.ERR_BAD_HANDLE
    args = so.AppendArgs()
    assert lib.relux_mla_append(None, C.byref(args)) == so.ERR_BAD_HANDLE


def test_struct_sizes_match_the_header(so):
    # relux_pool_params: 16 int32; relux_append_args / relux_attn_args as laid out by a C compiler
    assert C.sizeof(so.PoolParams) == 64
    import subprocess, tempfile, textwrap
    prog = textwrap.dedent("""
        #include <stdio.h>
        #include "relux_cuda.h"
        #include <stddef.h>
        int main(void){ printf("%zu %zu %zu %zu\\n", sizeof(relux_mla_expand_args), offsetof(relux_mla_expand_args, w_uk),
                               offsetof(relux_mla_expand_args, rows_total), offsetof(relux_mla_expand_args, rows_total_out));
                        printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(relux_read_rows_args), offsetof(relux_read_rows_args, dst_b),
                               sizeof(relux_stream_partition_args), offsetof(relux_stream_partition_args, chunk_off),
                               sizeof(relux_matmul_args), offsetof(relux_matmul_args, b), offsetof(relux_matmul_args, c),
                               sizeof(relux_mla_import_args), offsetof(relux_mla_import_args, q_proj), offsetof(relux_mla_import_args, dst));
                        printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(relux_pool_params), sizeof(relux_append_args),
                               sizeof(relux_attn_args), sizeof(relux_mla_layer_weights), sizeof(relux_mla_layer_args),
                               sizeof(relux_gqa_layer_weights), sizeof(relux_gqa_layer_args),
                               offsetof(relux_mla_layer_args, w), offsetof(relux_gqa_layer_args, w),
                               sizeof(relux_sampler_params), sizeof(relux_spec_accept_args), offsetof(relux_spec_accept_args, sampler),
                               offsetof(relux_spec_accept_args, next_token), sizeof(relux_sample_args),
                               offsetof(relux_sample_args, prev_tokens), offsetof(relux_sample_args, tokens)); return 0; }
    """)
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(prog)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    assert sizes[:4] == [C.sizeof(so.MlaExpandArgs), so.MlaExpandArgs.w_uk.offset, so.MlaExpandArgs.rows_total.offset,
                         so.MlaExpandArgs.rows_total_out.offset]
    sizes = sizes[4:]
    assert sizes[:10] == [C.sizeof(so.ReadRowsArgs), so.ReadRowsArgs.dst_b.offset, C.sizeof(so.StreamPartitionArgs),
                          so.StreamPartitionArgs.chunk_off.offset, C.sizeof(so.MatmulArgs), so.MatmulArgs.b.offset, so.MatmulArgs.c.offset,
                          C.sizeof(so.MlaImportArgs), so.MlaImportArgs.q_proj.offset, so.MlaImportArgs.dst.offset]
    sizes = sizes[10:]
    assert so.PoolParams.flags.offset == 40
    assert sizes == [C.sizeof(so.PoolParams), C.sizeof(so.AppendArgs), C.sizeof(so.AttnArgs), C.sizeof(so.MlaLayerWeights),
                     C.sizeof(so.MlaLayerArgs), C.sizeof(so.GqaLayerWeights), C.sizeof(so.GqaLayerArgs), so.MlaLayerArgs.w.offset,
                     so.GqaLayerArgs.w.offset, C.sizeof(so.SamplerParams), C.sizeof(so.SpecAcceptArgs),
                     so.SpecAcceptArgs.sampler.offset, so.SpecAcceptArgs.next_token.offset, C.sizeof(so.SampleArgs),
                     so.SampleArgs.prev_tokens.offset, so.SampleArgs.tokens.offset]


def test_no_gpu_means_a_clean_error(so):
    from tests.helpers import have_gpu
    if have_gpu():
        pytest.skip("a GPU is present")
    import relux_b200 as rb
    with pytest.raises(so.ReluxCudaError) as e:
        rb.Device(0)
    assert e.value.code in (so.ERR_NO_DEVICE, so.ERR_CUDA)


def test_every_entry_point_says_what_it_replaces():
    """Each declaration in the header stands under a comment that cites the reference (file.go:line) or says that the
    reference has no counterpart; a comment may head a group of consecutive declarations."""
    import re
    text = open(os.path.join(ROOT, "include", "relux_cuda.h")).read()
    text = re.sub(r"typedef struct \w+ \{.*?\} \w+;", "", text, flags=re.S)      # field comments are not entry-point comments
    missing = []
    for m in re.finditer(r"^int32_t (relux_\w+)\(", text, re.M):
        pre = text[:m.start()]
        end = pre.rfind("*/")
        begin = pre.rfind("/*", 0, end)
        block = pre[begin:end + 2] if end >= 0 else ""
        between = pre[end + 2:] if end >= 0 else pre
        only_decls = re.sub(r"int32_t relux_\w+\([^;]*\);", "", between).strip() == ""
        if not only_decls or not (re.search(r"\.go:\d", block) or "no counterpart" in block.lower()):
            missing.append(m.group(1))
    assert not missing, "entry points without a reference citation: %s" % missing
