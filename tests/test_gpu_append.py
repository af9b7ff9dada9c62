"""Append / page-table / readback parity on the GPU: cache rows must be BIT-EXACT with
BF16FromF32(row) of the oracle for any page permutation (calls go through the C ABI)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import relux_b200 as rb
    d = rb.Device(0)
    yield d
    d.close()


def _mla_pool(dev, B, pages_per, rng, dC=512, dHR=64, layers=2, P=64):
    import relux_b200 as rb
    from relux_b200 import lib as L
    from tests.helpers import permuted_tables
    pool = rb.Pool(dev, L.POOL_MLA, layers, B * pages_per + 3, P, B, pages_per, dC=dC, dHR=dHR)
    pool.set_tables(permuted_tables(rng, B, pages_per, B * pages_per + 3))
    return pool


@pytest.mark.parametrize("P", [64, 16])
@pytest.mark.parametrize("mem", ["host", "device"])
def test_mla_append_bit_exact_ragged(dev, oracle, P, mem):
    rng = np.random.default_rng(7)
    B, dC, dHR = 5, 512, 64
    pages_per = 5 if P == 64 else 20
    pool = _mla_pool(dev, B, pages_per, rng, P=P)
    ref_c = [np.zeros((0, dC), np.uint16) for _ in range(B)]
    ref_r = [np.zeros((0, dHR), np.uint16) for _ in range(B)]
    # step 0: ragged prefill crossing page boundaries; then single-token decodes; then ragged again with empties
    for n_new in ([63, 64, 65, 1, 130], None, None, [0, 3, 0, 70, 1]):
        nn = np.ones(B, np.int32) if n_new is None else np.array(n_new, np.int32)
        c = rng.standard_normal((int(nn.sum()), dC)).astype(np.float32)
        r = rng.standard_normal((int(nn.sum()), dHR)).astype(np.float32)
        for layer in (0, 1):
            if mem == "device":
                dc, dr = dev.upload(c), dev.upload(r)
                pool.append(layer, dc, dr, B, n_new=n_new)
                dev.sync(); dc.free(); dr.free()
            else:
                pool.append(layer, c, r, B, n_new=n_new)
        o = 0
        for b in range(B):
            ref_c[b] = np.concatenate([ref_c[b], oracle.bf16_from_f32(c[o:o + nn[b]])])
            ref_r[b] = np.concatenate([ref_r[b], oracle.bf16_from_f32(r[o:o + nn[b]])])
            o += nn[b]
    for layer in (0, 1):
        for b in range(B):
            T = pool.seq_len(layer, b)
            assert T == ref_c[b].shape[0]
            got_c, got_r = pool.read_rows(layer, b, 0, T)
            assert np.array_equal(got_c, ref_c[b]) and np.array_equal(got_r, ref_r[b])
    assert pool.status() == 0
    pool.destroy()


def test_mla_append_bf16_input_is_copied_bit_for_bit(dev, oracle):
    rng = np.random.default_rng(1)
    pool = _mla_pool(dev, 2, 2, rng)
    c = rng.integers(0, 0x7F00, (2, 512), dtype=np.uint16)   # arbitrary finite bf16 bit patterns
    r = rng.integers(0, 0x7F00, (2, 64), dtype=np.uint16)
    pool.append(0, c, r, 2)
    for b in range(2):
        gc, gr = pool.read_rows(0, b, 0, 1)
        assert np.array_equal(gc[0], c[b]) and np.array_equal(gr[0], r[b])
    pool.destroy()


def test_special_values_round_like_the_reference(dev, oracle):
    rng = np.random.default_rng(2)
    pool = _mla_pool(dev, 1, 1, rng)
    c = np.zeros((1, 512), np.float32)
    specials = np.array([0.0, -0.0, np.inf, -np.inf, 1.0, 1.00390625, 1.01171875, 3.3895314e38, 1e-40, -1e-40], np.float32)
    ties = np.array([0x3F808000, 0x3F818000, 0x3F808001, 0x7F7FFFFF], np.uint32).view(np.float32)
    c[0, :specials.size] = specials
    c[0, 16:16 + ties.size] = ties
    r = np.zeros((1, 64), np.float32)
    pool.append(0, c, r, 1)
    gc, _ = pool.read_rows(0, 0, 0, 1)
    assert np.array_equal(gc[0], oracle.bf16_from_f32(c[0]))
    pool.destroy()


@pytest.mark.parametrize("layout", ["token", "head"])
def test_gqa_append_bit_exact(dev, oracle, layout):
    import relux_b200 as rb
    from relux_b200 import lib as L
    from tests.helpers import permuted_tables
    rng = np.random.default_rng(3)
    B, Hkv, D, P, pages_per = 3, 8, 128, 64, 3
    pool = rb.Pool(dev, L.POOL_GQA, 2, B * pages_per, P, B, pages_per, num_kv_heads=Hkv, head_dim=D)
    pool.set_tables(permuted_tables(rng, B, pages_per))
    refK = [np.zeros((0, Hkv, D), np.uint16) for _ in range(B)]
    refV = [np.zeros((0, Hkv, D), np.uint16) for _ in range(B)]
    for n_new in ([70, 1, 64], None, [4, 0, 2]):
        nn = np.ones(B, np.int32) if n_new is None else np.array(n_new, np.int32)
        K = rng.standard_normal((int(nn.sum()), Hkv, D)).astype(np.float32)
        V = rng.standard_normal((int(nn.sum()), Hkv, D)).astype(np.float32)
        if layout == "head":   # per sequence [Hkv][n_new][D], the reference's tensor layout
            o, ks, vs = 0, [], []
            for b in range(B):
                ks.append(np.ascontiguousarray(K[o:o + nn[b]].transpose(1, 0, 2)).ravel())
                vs.append(np.ascontiguousarray(V[o:o + nn[b]].transpose(1, 0, 2)).ravel())
                o += nn[b]
            Ka, Va = np.concatenate(ks), np.concatenate(vs)
            pool.append(1, Ka, Va, B, n_new=nn, layout=L.LAYOUT_HEAD_MAJOR)
        else:
            pool.append(1, K, V, B, n_new=n_new)
        o = 0
        for b in range(B):
            refK[b] = np.concatenate([refK[b], oracle.bf16_from_f32(K[o:o + nn[b]])])
            refV[b] = np.concatenate([refV[b], oracle.bf16_from_f32(V[o:o + nn[b]])])
            o += nn[b]
    for b in range(B):
        T = pool.seq_len(1, b)
        assert T == refK[b].shape[0] and pool.seq_len(0, b) == 0
        gk, gv = pool.read_rows(1, b, 0, T)
        assert np.array_equal(gk, refK[b]) and np.array_equal(gv, refV[b])
    assert pool.status() == 0
    pool.destroy()


def test_kvcache_object_matches_reference_tests(dev, oracle):
    """The reference's own KVCache tests (kvcache_test.go:16-66, 87-107) replayed on the device cache."""
    import relux_b200 as rb
    c = rb.KVCache(dev, 2, 64, 2, 8)
    assert c.TotalLen(0) == 0 and c.View(0) == (None, None)
    k = np.arange(1, 17, dtype=np.float32).reshape(1, 2, 1, 8)
    v = np.arange(17, 33, dtype=np.float32).reshape(1, 2, 1, 8)
    c.Append(0, k, v)
    assert c.TotalLen(0) == 1 and c.TotalLen(1) == 0
    ck, cv = c.View(0)
    assert ck.shape == (1, 2, 1, 8)
    assert np.array_equal(oracle.f32_from_bf16(ck), k) and np.array_equal(oracle.f32_from_bf16(cv), v)
    # grow: one head, 1 token then 2 tokens -> concatenation (kvcache_test.go:42-66)
    c1 = rb.KVCache(dev, 1, 16, 1, 8)
    a = np.arange(1, 9, dtype=np.float32).reshape(1, 1, 1, 8)
    b = np.arange(9, 25, dtype=np.float32).reshape(1, 1, 2, 8)
    c1.Append(0, a, a)
    c1.Append(0, b, b)
    assert c1.TotalLen(0) == 3
    ck, _ = c1.View(0)
    assert oracle.f32_from_bf16(ck).ravel().tolist() == list(range(1, 25))
    c1.Reset()
    assert c1.TotalLen(0) == 0 and c1.View(0) == (None, None)
    with pytest.raises(IndexError):
        c.Append(5, k, v)
    c.close(); c1.close()


def test_overflow_and_bad_page_are_reported_not_faulted(dev):
    import relux_b200 as rb
    from relux_b200 import lib as L
    pool = rb.Pool(dev, L.POOL_MLA, 1, 4, 64, 2, 2, dC=64, dHR=16)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.set_tables(np.array([[0, 9], [1, 2]], np.int32))
    assert e.value.code == L.ERR_BAD_PAGE
    pool.set_tables(np.array([[0, 3], [1, 2]], np.int32))
    c = np.zeros((2 * 128, 64), np.float32)
    r = np.zeros((2 * 128, 16), np.float32)
    pool.append(0, c, r, 2, n_new=[128, 128])
    with pytest.raises(L.ReluxCudaError) as e:   # the reference panics: "overflow: total=128 + newLen=1 > capacity=128"
        pool.append(0, c[:2], r[:2], 2)
    assert e.value.code == L.ERR_OVERFLOW and "overflow" in str(e.value)
    assert pool.seq_len(0, 0) == 128
    assert pool.status() == 0
    pool.destroy()


def test_library_owned_sequences_and_exhaustion(dev):
    import relux_b200 as rb
    from relux_b200 import lib as L
    pool = rb.Pool(dev, L.POOL_MLA, 1, 4, 64, 3, 4, dC=64, dHR=16)
    a = pool.seq_alloc(100)
    b = pool.seq_alloc(128)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.seq_alloc(1)
    assert e.value.code == L.ERR_POOL_EXHAUSTED
    pool.seq_free(a)
    c = pool.seq_alloc(65)
    assert c == a
    x = np.ones((1, 64), np.float32); y = np.ones((1, 16), np.float32)
    pool.append(0, x, y, 1, seq_ids=[b])
    assert pool.seq_len(0, b) == 1 and pool.seq_len(0, c) == 0
    pool.reset()
    assert pool.seq_len(0, b) == 0
    pool.destroy()


def test_sequence_grows_page_by_page(dev, oracle):
    """relux_seq_extend: a sequence starts with one page and takes more from the free list as it fills; rows already
    cached stay bit-exact, and the free list is honoured."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    rng = np.random.default_rng(71)
    pool = rb.Pool(dev, L.POOL_MLA, 1, 5, 64, 2, 4, dC=64, dHR=16)
    s = pool.seq_alloc(64)
    other = pool.seq_alloc(64)
    c = rng.standard_normal((200, 64), dtype=np.float32)
    r = rng.standard_normal((200, 16), dtype=np.float32)
    pool.append(0, c[:64], r[:64], 1, seq_ids=[s], n_new=[64])
    with pytest.raises(L.ReluxCudaError) as e:       # the page is full
        pool.append(0, c[64:65], r[64:65], 1, seq_ids=[s])
    assert e.value.code == L.ERR_OVERFLOW
    pool.seq_extend(s, 200)                           # 4 pages = 3 more of the 3 free ones
    pool.append(0, c[64:200], r[64:200], 1, seq_ids=[s], n_new=[136])
    gc, gr = pool.read_rows(0, s, 0, 200)
    assert np.array_equal(gc, oracle.bf16_from_f32(c)) and np.array_equal(gr, oracle.bf16_from_f32(r))
    pool.seq_extend(s, 100)                           # never shrinks
    assert pool.seq_len(0, s) == 200
    with pytest.raises(L.ReluxCudaError) as e:
        pool.seq_extend(other, 128)                   # no free page left
    assert e.value.code == L.ERR_POOL_EXHAUSTED
    with pytest.raises(L.ReluxCudaError) as e:
        pool.seq_extend(s, 64 * 5)                    # beyond max_pages_per_seq
    assert e.value.code == L.ERR_OVERFLOW
    assert pool.status() == 0
    pool.destroy()


def test_a_sequence_named_twice_is_refused_whatever_the_batch_size(dev):
    """Two blocks of one append would write the same rows and the cursor would move twice: refused on the host, for
    small batches and for batches of hundreds of sequences alike."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    n = 300
    pool = rb.Pool(dev, L.POOL_MLA, 1, n, 64, n, 1, dC=64, dHR=16)
    pool.set_tables(np.arange(n, dtype=np.int32).reshape(n, 1))
    c = np.ones((n, 64), np.float32); r = np.ones((n, 16), np.float32)
    for ids in ([0, 1, 1], list(range(n - 1)) + [17]):
        with pytest.raises(L.ReluxCudaError) as e:
            pool.append(0, c[:len(ids)], r[:len(ids)], len(ids), seq_ids=ids)
        assert e.value.code == L.ERR_INVALID_ARG and "twice" in str(e.value)
    assert all(pool.seq_len(0, s) == 0 for s in (0, 1, 17))
    pool.append(0, c, r, n, seq_ids=list(range(n))[::-1])   # a permutation is fine
    assert pool.seq_len(0, 17) == 1 and pool.status() == 0
    pool.destroy()


def test_misaligned_device_pointers_are_refused_before_any_launch(dev):
    """The kernels read device inputs with 16-byte vector loads; an offset pointer would fault.  It is refused."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    pool = rb.Pool(dev, L.POOL_MLA, 1, 2, 64, 1, 2, dC=64, dHR=16)
    pool.set_tables(np.arange(2, dtype=np.int32).reshape(1, 2))
    buf = dev.alloc(4096, L.DTYPE_BF16)
    n0 = dev.launch_count()
    with pytest.raises(L.ReluxCudaError) as e:
        pool.append(0, buf.ptr + 2, buf.ptr + 1024, 1, dtype=L.DTYPE_BF16)
    assert e.value.code == L.ERR_INVALID_ARG and "aligned" in str(e.value)
    assert dev.launch_count() == n0 and pool.seq_len(0, 0) == 0
    pool.append(0, buf.ptr + 16, buf.ptr + 1024, 1, dtype=L.DTYPE_BF16)   # 16-byte aligned offsets are fine
    w = dev.alloc(64 * 2 * 32 * 2 + 64, L.DTYPE_BF16)
    q = dev.alloc(8192, L.DTYPE_F32)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.decode(0, 1, q.ptr + 4, q.ptr + 4096, 2, 32, 0.1, q_rope=q.ptr + 2048, w_uk=w, w_uv=w, q_dtype=L.DTYPE_F32, out_dtype=L.DTYPE_F32)
    assert e.value.code == L.ERR_INVALID_ARG
    assert pool.status() == 0
    for b in (buf, w, q):
        b.free()
    pool.destroy()


def test_a_wait_that_nobody_answers_gives_up_and_reports(dev):
    """Every device-side wait of the library is bounded.  The self test runs the same polling loop on a barrier nobody
    arrives at, with a limit of a few thousand polls: the kernel returns, the status word says RELUX_ERR_TIMEOUT, and the
    context is as usable afterwards as before."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    pool = rb.Pool(dev, L.POOL_MLA, 1, 2, 64, 1, 2, dC=64, dHR=16)
    pool.set_tables(np.arange(2, dtype=np.int32).reshape(1, 2))
    assert pool.status() == 0
    pool.selftest_wait(3000)
    assert pool.status() == L.ERR_TIMEOUT
    assert pool.status() == 0   # reading clears it
    pool.append(0, np.ones((1, 64), np.float32), np.ones((1, 16), np.float32), 1)
    assert pool.seq_len(0, 0) == 1 and pool.status() == 0
    pool.destroy()


def test_one_owner_of_the_pages_per_pool(dev):
    """Caller-made page tables and the library's free list do not mix on one pool, and a page may be mapped once."""
    import relux_b200 as rb
    from relux_b200 import lib as L
    pool = rb.Pool(dev, L.POOL_MLA, 1, 4, 64, 2, 2, dC=64, dHR=16)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.set_tables(np.array([[0, 1], [1, 2]], np.int32))
    assert e.value.code == L.ERR_BAD_PAGE and "twice" in str(e.value)
    pool.set_tables(np.array([[0, 1], [3, 2]], np.int32))
    with pytest.raises(L.ReluxCudaError) as e:
        pool.seq_alloc(10)
    assert e.value.code == L.ERR_INVALID_ARG
    pool.destroy()
    pool = rb.Pool(dev, L.POOL_MLA, 1, 4, 64, 2, 2, dC=64, dHR=16)
    pool.seq_alloc(10)
    with pytest.raises(L.ReluxCudaError) as e:
        pool.set_tables(np.array([[0, 1], [3, 2]], np.int32))
    assert e.value.code == L.ERR_INVALID_ARG
    pool.destroy()
