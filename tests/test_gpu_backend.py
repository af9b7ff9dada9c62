"""The matmul of the compute backend (ComputeBackend.MatMulFloat32 as matmulBatched3D calls it) and the weight import,
through the C ABI, against the CPU restatement."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


@pytest.fixture(scope="module")
def pool(dev):
    import relux_b200 as rb
    from relux_b200 import lib as L
    p = rb.Pool(dev, L.POOL_MLA, 1, 2, 64, 1, 2, dC=64, dHR=16)   # the calls need a pool for its stream and scratch
    yield p
    p.destroy()


@pytest.mark.parametrize("M", [1, 64, 129, 512])
def test_matmul_reference_is_bit_exact_and_fast_within_tolerance(dev, pool, oracle, M):
    """REFERENCE: the k-ascending unfused chain of matmul.go:15-27, bit for bit.  FAST: bf16 tensor-core GEMM, float32
    accumulation: within 2^-8 relative of the row norms (A is rounded to bf16)."""
    from relux_b200 import lib as L
    rng = np.random.default_rng(100 + M)
    K, N = 264, 392   # not multiples of the 128 x 128 x 64 tile: the edges are exercised
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = oracle.bf16_from_f32((rng.standard_normal((K, N)) * 0.05).astype(np.float32))
    d_w = dev.upload(w)
    ref = oracle.matmul_batched3d(a, w)
    out = pool.matmul(a, d_w, N, mode=L.ATTN_REFERENCE)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    fast = pool.matmul(a, d_w, N, mode=L.ATTN_FAST)
    wf = oracle.f32_from_bf16(w).astype(np.float64)
    bound = 2.0 ** -8 * (np.abs(a).astype(np.float64) @ np.abs(wf)) + 1e-5
    assert (np.abs(fast - ref) <= bound).all()
    assert np.abs(fast - ref).max() <= 2e-2
    # device-resident A and C
    d_a, d_c = dev.upload(a), dev.alloc(M * N * 4, L.DTYPE_F32)
    import ctypes as C
    args = L.MatmulArgs(m=M, k=K, n=N, mode=L.ATTN_REFERENCE, a=d_a.ptr, a_mem=L.MEM_DEVICE, c_mem=L.MEM_DEVICE, b=d_w.ptr, c=d_c.ptr)
    L.check(pool.lib.relux_matmul_f32_bf16(pool.h, C.byref(args)))
    assert np.array_equal(d_c.download((M, N), np.float32).view(np.uint32), ref.view(np.uint32))
    for b in (d_w, d_a, d_c):
        b.free()
    assert pool.status() == 0


def test_matmul_refuses_what_it_cannot_do(dev, pool, oracle):
    from relux_b200 import lib as L
    a = np.ones((2, 12), np.float32)
    d_w = dev.upload(np.zeros((12, 20), np.uint16))
    with pytest.raises(L.ReluxCudaError) as e:   # K, N not multiples of 8: no tensor-core path, and no silent fallback
        pool.matmul(a, d_w, 20, mode=L.ATTN_FAST)
    assert e.value.code == L.ERR_UNSUPPORTED
    out = pool.matmul(a, d_w, 20, mode=L.ATTN_REFERENCE)
    assert (out == 0).all()
    import ctypes as C
    args = L.MatmulArgs(m=2, k=12, n=20, mode=L.ATTN_REFERENCE, a=a.ctypes.data, a_mem=L.MEM_HOST, c_mem=L.MEM_HOST, b=d_w.ptr + 2,
                        c=out.ctypes.data)
    assert pool.lib.relux_matmul_f32_bf16(pool.h, C.byref(args)) == L.ERR_INVALID_ARG   # misaligned device pointer
    d_w.free()


@pytest.mark.parametrize("fused,dtype", [(True, np.float32), (False, np.float32), (True, np.uint16)])
def test_mla_weight_import_is_bit_exact(dev, pool, oracle, fused, dtype):
    """Split + transpose of one layer's checkpoint tensors on the device against the numpy restatement, bit for bit:
    float32 sources (rounded with BF16FromF32) and bf16 sources (moved as they are)."""
    rng = np.random.default_rng(7)
    D, H, dn, dr, dv, dC = 96, 6, 24, 8, 40, 56   # odd sizes: tiles of 32 have ragged edges

    def tensor(rows, cols):
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        return x if dtype == np.float32 else oracle.bf16_from_f32(x)

    src = {"q_proj": tensor(H * (dn + (dr if fused else 0)), D), "kv_a_proj_with_mqa": tensor(dC + (dr if fused else 0), D),
           "kv_b_proj": tensor(H * (dn + dv), dC), "o_proj": tensor(D, H * dv)}
    if not fused:
        src["q_pe_proj"] = tensor(H * dr, D)
        src["k_pe_proj"] = tensor(dr, D)
    want = oracle.import_mla_weights(D, H, dn, dr, dv, dC, fused_rope=fused, **src)
    shapes = {"w_q": (D, H * dn), "w_qr": (D, H * dr), "w_dkv": (D, dC), "w_kr": (D, dr), "w_uk": (dC, H * dn), "w_uv": (dC, H * dv),
              "w_o": (H * dv, D)}
    dst = {k: dev.alloc(int(np.prod(s)) * 2) for k, s in shapes.items()}
    pool.import_mla_weights(D, H, dn, dr, dv, dC, dst, fused_rope=fused, **src)
    for k, shp in shapes.items():
        got = dst[k].download(shp, np.uint16)
        assert got.shape == want[k].shape and np.array_equal(got, want[k]), k
        dst[k].free()
    assert pool.status() == 0


def test_imported_weights_feed_the_layer_call(dev, oracle):
    """A layer step with weights that came through the import equals one with weights uploaded in relux's layout."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(8)
    D, H, dC, dr = 128, 4, 64, 16
    dn = dv = D // H
    pool = rb.Pool(dev, L.POOL_MLA, 1, 4, 64, 1, 4, dC=dC, dHR=dr)
    pool.set_tables(np.arange(4, dtype=np.int32).reshape(1, 4))
    ck = {"q_proj": rng.standard_normal((H * (dn + dr), D)).astype(np.float32) * 0.1,
          "kv_a_proj_with_mqa": rng.standard_normal((dC + dr, D)).astype(np.float32) * 0.1,
          "kv_b_proj": rng.standard_normal((H * (dn + dv), dC)).astype(np.float32) * 0.1,
          "o_proj": rng.standard_normal((D, H * dv)).astype(np.float32) * 0.1}
    want = oracle.import_mla_weights(D, H, dn, dr, dv, dC, fused_rope=True, **ck)
    direct = {k: dev.upload(v) for k, v in want.items()}
    imported = {k: dev.alloc(v.nbytes) for k, v in want.items()}
    pool.import_mla_weights(D, H, dn, dr, dv, dC, imported, fused_rope=True, **ck)
    x = rng.standard_normal((1, 5, D)).astype(np.float32)
    y1, y2 = np.empty_like(x), np.empty_like(x)
    pool.forward_cached(0, 1, x, y1, direct, D, H, q_tokens=5, mode=L.ATTN_REFERENCE)
    pool.set_len(-1, [0])
    pool.forward_cached(0, 1, x, y2, imported, D, H, q_tokens=5, mode=L.ATTN_REFERENCE)
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32)) and np.isfinite(y1).all() and np.abs(y1).max() > 0
    for d in (direct, imported):
        for b in d.values():
            b.free()
    pool.destroy()
