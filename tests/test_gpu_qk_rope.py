"""q/k RMSNorm + NeoX RoPE (YaRN) + paged-KV write: CUDA path vs the CPU oracle.

Both sides get the SAME inv_freq table, so what remains is cosf/sinf of the
device vs the C library (<= 3 FP32 ulp on each product).  Tolerance: one BF16
ulp at the magnitude of the largest of the two rotation terms |n1*c|, |n2*s|
and the result itself — the rotation is a sum/difference of two such terms, so
where no cancellation happens this is 1 BF16 ulp of the result.  Paged addressing is checked byte for byte:
every K/V row must sit at the address recomputed on the host and every other
byte of the 0xFF-poisoned pools must be untouched."""
import importlib

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
wl = importlib.import_module("axiom-kernel_b200.workloads")


def tolerance(q_in, gamma, inv_freq, positions, rope_dim, mscale, eps=1e-6):
    """Per-element bound: 1 BF16 ulp at max(|n1 c|, |n2 s|, |result|) (FP64 evaluation)."""
    x = wl.from_bf16_bits(q_in).astype(np.float64)
    g = wl.from_bf16_bits(gamma).astype(np.float64)
    n = x / np.sqrt((x ** 2).mean(axis=-1, keepdims=True) + eps) * g
    half = rope_dim // 2
    ang = positions.astype(np.float32)[:, None] * inv_freq[None, :]
    c = (np.cos(ang.astype(np.float64)) * mscale)[:, None, :]
    s = (np.sin(ang.astype(np.float64)) * mscale)[:, None, :]
    mag = np.abs(n).copy()
    a, b = n[..., :half], n[..., half:rope_dim]
    mag[..., :half] = np.maximum(np.maximum(np.abs(a * c), np.abs(b * s)), np.abs(a * c - b * s))
    mag[..., half:rope_dim] = np.maximum(np.maximum(np.abs(a * s), np.abs(b * c)), np.abs(a * s + b * c))
    return ol.bf16_ulp(mag.astype(np.float32)) * np.float32(1.01)


def run_case(axk, tokens, q_heads, k_heads, head_dim, rope_dim, *, n_blocks=64, block_tokens=16, n_layers=2, layer=1,
             pool_pad=0, ring=True, per_token=False, with_v=True, theta=1e6, factor=4.0, ctx=32768.0, max_base=100000,
             seed=3, fp8_cache=False, q_mode="inplace"):
    import torch
    from gpu_util import Guarded, dev, host, sync

    q, k, v, qg, kg, positions, table = wl.qk_inputs_np(tokens, q_heads, k_heads, head_dim, n_blocks, seed, max_base)
    if per_token:
        rng = np.random.default_rng(seed + 1)
        if tokens <= 64:
            table = np.stack([rng.permutation(n_blocks).astype(np.int32) for _ in range(tokens)])
            positions = rng.integers(0, n_blocks * block_tokens, tokens).astype(np.uint32)
        else:  # many tokens: one permutation in every row and distinct positions, so no two tokens share a cell
            table = np.tile(rng.permutation(n_blocks).astype(np.int32), (tokens, 1))
            positions = rng.permutation(n_blocks * block_tokens)[:tokens].astype(np.uint32)
    inv_freq = ol.yarn_inv_freq(theta, factor, ctx, 32.0, 1.0, rope_dim) if rope_dim else np.zeros(1, np.float32)
    mscale = float(ol.o().axo_yarn_mscale(factor))
    kv_dim = k_heads * head_dim
    pool_stride = kv_dim + pool_pad
    pool_elems = n_blocks * n_layers * block_tokens * pool_stride
    cell = 1 if fp8_cache else 2  # bytes per cache element
    k_pool, v_pool = Guarded(pool_elems * cell), Guarded(pool_elems * cell)
    k_out = Guarded(tokens * kv_dim * 2)
    # q_mode: "inplace" rewrites Q; "out" leaves Q alone and writes q_out; "interleaved" reads the query halves of a
    # [tokens][heads][2 * head_dim] q-projection output (gate values behind every head) and writes q_out
    q_source = q
    if q_mode == "interleaved":
        gate_rng = np.random.default_rng(seed + 17)
        q_source = np.concatenate([q, gate_rng.integers(0, 1 << 16, q.shape).astype(np.uint16)], axis=-1)
    q_out = Guarded(tokens * q_heads * head_dim * 2) if q_mode != "inplace" else None
    qd, kd, vd = dev(q_source), dev(k), dev(v)
    # every device tensor is named: the argument struct only carries raw addresses
    qgd, kgd, fd, pd, td = dev(qg), dev(kg), dev(inv_freq), dev(positions), dev(table)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = ((axk.QK_FLAG_RING if ring else 0) | (axk.QK_FLAG_PER_TOKEN_TABLE if per_token else 0) |
             (axk.QK_FLAG_CACHE_E4M3 if fp8_cache else 0) |
             (axk.QK_FLAG_Q_GATE_INTERLEAVED if q_mode == "interleaved" else 0))
    args = axk.make_qk_args(tokens=tokens, q_heads=q_heads, k_heads=k_heads, head_dim=head_dim, rope_dim=rope_dim,
                            flags=flags, eps=1e-6, mscale=mscale, block_tokens=block_tokens, n_layers=n_layers,
                            layer=layer, pool_stride=pool_stride, tbl_stride=table.shape[1], n_blocks=n_blocks,
                            q=qd, k=kd, v=vd if with_v else None, q_gamma=qgd, k_gamma=kgd,
                            inv_freq=fd, positions=pd, block_tables=td,
                            k_pool=k_pool.ptr, v_pool=v_pool.ptr if with_v else None, k_out=k_out.ptr,
                            status_word=status, q_out=q_out.ptr if q_out else None)
    rc = axk.qk_norm_rope_paged(0, args)
    sync()
    assert rc == axk.AXIOM_OK
    assert k_pool.guards_intact() and v_pool.guards_intact() and k_out.guards_intact()
    if q_out:
        assert q_out.guards_intact()
        assert np.array_equal(host(qd, np.uint16).reshape(q_source.shape), q_source)  # the source is only read

    # oracle on identical inputs, with poisoned pools of its own
    o_kpool = np.full(pool_elems, 0xFFFF, np.uint16)
    o_vpool = np.full(pool_elems, 0xFFFF, np.uint16)
    want_q, want_k, want_status = ol.qk_norm_rope_paged(
        q, k, v if with_v else None, qg, kg, inv_freq, positions, table, rope_dim=rope_dim, eps=1e-6, mscale=mscale,
        block_tokens=block_tokens, n_layers=n_layers, layer=layer, pool_stride=pool_stride, n_blocks=n_blocks,
        ring=ring, per_token_table=per_token, k_pool=o_kpool, v_pool=o_vpool if with_v else None, want_k_out=True)
    got_q = (q_out.payload(np.uint16) if q_out else host(qd, np.uint16)).reshape(q.shape)
    got_k = k_out.payload(np.uint16).reshape(k.shape)
    assert int(status.item()) == want_status

    for got, want, src, gamma in ((got_q, want_q, q, qg), (got_k, want_k, k, kg)):
        a, b = wl.from_bf16_bits(got), wl.from_bf16_bits(want)
        tol = tolerance(src, gamma, inv_freq, positions, rope_dim, mscale)
        assert np.all(np.abs(a - b) <= tol)
        assert np.mean(got != want) < 0.02
        if rope_dim < head_dim:  # pass-through dims have no transcendental: bit-exact
            assert np.array_equal(got[..., rope_dim:], want[..., rope_dim:])

    # paged scatter: exactly the oracle's cells were written, with this kernel's own K rows; V is a copy
    got_kpool, got_vpool = k_pool.payload(np.uint8 if fp8_cache else np.uint16), v_pool.payload(np.uint8 if fp8_cache else np.uint16)
    written = o_kpool != 0xFFFF
    expect_kpool = np.full(pool_elems, 0xFFFF, np.uint16)
    for t in range(tokens):
        pos = int(positions[t])
        lb = (pos // block_tokens) % table.shape[1] if ring else pos // block_tokens
        if lb >= table.shape[1]:
            continue
        pb = int(table[t if per_token else 0, lb])
        if pb < 0 or pb >= n_blocks:
            continue
        base = ((pb * n_layers + layer) * block_tokens + pos % block_tokens) * pool_stride
        expect_kpool[base:base + kv_dim] = got_k[t].reshape(-1)
    if fp8_cache:
        # E4M3 cache: every written cell is the saturating E4M3 code (scale 1) of the BF16 value, the rest keeps
        # the guard pattern 0xFF
        assert np.array_equal(got_kpool, np.where(written, ol.bf16_to_e4m3_scale1(expect_kpool), 0xFF).astype(np.uint8))
        if with_v:
            v_written = o_vpool != 0xFFFF
            assert np.array_equal(got_vpool, np.where(v_written, ol.bf16_to_e4m3_scale1(o_vpool), 0xFF).astype(np.uint8))
        else:
            assert v_pool.untouched()
        return got_q, got_k
    assert np.array_equal(got_kpool, expect_kpool)
    assert np.array_equal(got_kpool != 0xFFFF, written)
    if with_v:
        assert np.array_equal(got_vpool, o_vpool)  # V is copied unchanged: bit-exact
    else:
        assert v_pool.untouched()
    return got_q, got_k


@pytest.mark.parametrize("tokens", [1, 2, 7, 8, 9, 15, 16, 17, 64])
def test_config3_geometry_small(axk, cuda_device, tokens):
    run_case(axk, tokens, 64, 8, 128, 128, n_blocks=4096, n_layers=1, layer=0)


@pytest.mark.parametrize("q_heads,k_heads,head_dim,rope_dim", [(24, 4, 256, 64), (40, 8, 128, 128), (3, 1, 64, 64),
                                                                (5, 2, 64, 32), (2, 2, 256, 256), (1, 1, 128, 16),
                                                                (16, 2, 128, 0)])
def test_other_geometries(axk, cuda_device, q_heads, k_heads, head_dim, rope_dim):
    run_case(axk, 33, q_heads, k_heads, head_dim, rope_dim, theta=1e7, ctx=262144.0)


def test_pool_stride_padding_layers_and_no_v(axk, cuda_device):
    run_case(axk, 40, 8, 2, 128, 128, n_layers=3, layer=2, pool_pad=64, n_blocks=32, max_base=300)
    run_case(axk, 40, 8, 2, 128, 128, with_v=False, n_blocks=32, max_base=300)


def test_per_token_tables_decode_batch(axk, cuda_device):
    run_case(axk, 64, 64, 8, 128, 128, per_token=True, n_blocks=128)


@pytest.mark.parametrize("q_heads,k_heads,head_dim,rope_dim", [(64, 8, 128, 128), (24, 4, 256, 64), (40, 8, 128, 128),
                                                                (6, 2, 64, 32), (16, 2, 128, 0), (5, 1, 64, 64)])
def test_streaming_kernel_geometries(axk, cuda_device, q_heads, k_heads, head_dim, rope_dim):
    """Token counts of two or more per SM take the persistent streaming kernel (or, for shapes it does not
    cover, the per-token kernel): 148 * 4 + 5 tokens leave the teams ragged tails."""
    run_case(axk, 597, q_heads, k_heads, head_dim, rope_dim, n_blocks=1024, n_layers=2, layer=1, theta=1e7,
             ctx=262144.0, max_base=4000)


def test_streaming_kernel_variants(axk, cuda_device):
    run_case(axk, 400, 8, 2, 128, 128, n_layers=3, layer=2, pool_pad=64, n_blocks=64, max_base=300)
    run_case(axk, 400, 8, 2, 128, 128, with_v=False, n_blocks=64, max_base=300)
    run_case(axk, 333, 64, 8, 128, 128, per_token=True, n_blocks=128)
    run_case(axk, 300, 16, 4, 128, 128, ring=False, n_blocks=16, max_base=100)  # half the tokens fall off the table


@pytest.mark.parametrize("tokens", [9, 64, 333, 597])
def test_e4m3_cache_flavour(axk, cuda_device, tokens):
    """K and V go to an FP8 cache as E4M3 codes at scale 1; Q and k_out stay BF16."""
    run_case(axk, tokens, 64, 8, 128, 128, n_blocks=1024, n_layers=1, layer=0, fp8_cache=True, max_base=4000)
    run_case(axk, tokens, 24, 4, 256, 64, n_blocks=256, n_layers=2, layer=1, pool_pad=64, fp8_cache=True, max_base=900,
             theta=1e7, ctx=262144.0)
    run_case(axk, tokens, 8, 2, 128, 128, n_blocks=64, fp8_cache=True, with_v=False, max_base=300)


@pytest.mark.parametrize("q_mode", ["out", "interleaved"])
@pytest.mark.parametrize("tokens", [1, 9, 64, 333, 597])
def test_query_written_out_of_place_and_gate_interleaved_source(axk, cuda_device, tokens, q_mode):
    """q_out_bf16 (per-token kernel below 296 tokens, streaming kernel above) and the q-projection layout with the
    gate values behind every head: same results as the packed in-place call, source untouched."""
    run_case(axk, tokens, 64, 8, 128, 128, n_blocks=1024, n_layers=1, layer=0, max_base=4000, q_mode=q_mode)
    run_case(axk, tokens, 24, 4, 256, 64, n_blocks=256, n_layers=2, layer=1, max_base=900, theta=1e7, ctx=262144.0,
             q_mode=q_mode)
    run_case(axk, tokens, 5, 1, 64, 64, n_blocks=256, max_base=900, q_mode=q_mode, fp8_cache=(q_mode == "out"))
    if tokens >= 296:
        # more heads than one box of a tensor map can hold (256): the streaming kernel fetches the heads one by one
        run_case(axk, tokens, 320, 64, 64, 64, n_blocks=256, max_base=900, q_mode=q_mode)


def test_interleaved_source_matches_packed_call_bitwise(axk, cuda_device):
    import torch
    from gpu_util import dev, sync

    tokens = 1024
    q, k, v, qg, kg, positions, table = wl.qk_inputs_np(tokens, 64, 8, 128, 4096, seed=5)
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    qgd, kgd, fd, td, pd, kd = dev(qg), dev(kg), dev(inv_freq), dev(table), dev(positions), dev(k)
    gate = np.random.default_rng(0).integers(0, 1 << 16, q.shape).astype(np.uint16)
    packed, source = dev(q), dev(np.concatenate([q, gate], axis=-1))
    out = torch.zeros(tokens * 8192, dtype=torch.int16, device="cuda")
    results = []
    for flags, qbuf, q_out in ((axk.QK_FLAG_RING, packed, None),
                               (axk.QK_FLAG_RING | axk.QK_FLAG_Q_GATE_INTERLEAVED, source, out)):
        ko = torch.zeros(tokens * 1024, dtype=torch.int16, device="cuda")
        args = axk.make_qk_args(tokens=tokens, q_heads=64, k_heads=8, head_dim=128, rope_dim=128, flags=flags, eps=1e-6,
                                mscale=mscale, block_tokens=16, n_layers=1, layer=0, pool_stride=1024, tbl_stride=4096,
                                n_blocks=4096, q=qbuf, k=kd, q_gamma=qgd, k_gamma=kgd, inv_freq=fd, positions=pd,
                                block_tables=td, k_out=ko, q_out=q_out)
        assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
        sync()
        results.append(((q_out if q_out is not None else qbuf).cpu().numpy().view(np.uint16).reshape(-1), ko.cpu().numpy()))
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])
    assert np.array_equal(source.cpu().numpy().view(np.uint16).reshape(tokens, 64, 256)[..., 128:], gate)
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0


def test_interleaved_source_needs_q_out(axk, cuda_device):
    import torch

    buf = torch.zeros(1 << 16, dtype=torch.int16, device="cuda")
    f = torch.zeros(64, dtype=torch.float32, device="cuda")
    p = torch.zeros(4, dtype=torch.int32, device="cuda")
    args = axk.make_qk_args(tokens=4, q_heads=4, k_heads=1, head_dim=128, rope_dim=128,
                            flags=axk.QK_FLAG_Q_GATE_INTERLEAVED, eps=1e-6, mscale=1.0, block_tokens=16, n_layers=1,
                            layer=0, pool_stride=128, tbl_stride=1, n_blocks=1, q=buf, k=buf, q_gamma=buf, k_gamma=buf,
                            inv_freq=f, positions=p, k_out=buf)
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("tokens", [70, 600])
def test_e4m3_page_records_of_the_kv_tier(axk, cuda_device, tokens):
    """The reference's tier record (include/axiom/qwen38_kv_tier.h:9-19; written on the device by
    qwen38_stream_store_kv_page_kernel, src/axiom_qwen38_attention.cu:1438-1449): a 256-token page is E4M3
    K[256][kv_dim] followed by E4M3 V[256][kv_dim], 512 KiB at kv_dim 1024.  The paged addressing of the q/k call
    expresses it with block_tokens = 256, two "layers" per page (the K half and the V half) and the V pool
    pointer advanced by one half: every record is then produced by the kernel itself."""
    import torch
    from gpu_util import Guarded, dev, sync

    q_heads, k_heads, D, rope_dim, pages = 24, 4, 256, 64, 4
    kv_dim, page_tokens = k_heads * D, 256
    half_bytes = page_tokens * kv_dim
    q, k, v, qg, kg, _, _ = wl.qk_inputs_np(tokens, q_heads, k_heads, D, pages, seed=21)
    positions = (1000 + np.arange(tokens)).astype(np.uint32)
    table = np.array([[2, 0, 3, 1]], np.int32)
    inv_freq = ol.yarn_inv_freq(1e7, 4.0, 262144.0, 32.0, 1.0, rope_dim)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    records = Guarded(pages * 2 * half_bytes)
    qd, kd, vd, qgd, kgd, fd, pd, td = dev(q), dev(k), dev(v), dev(qg), dev(kg), dev(inv_freq), dev(positions), dev(table)
    k_out = torch.zeros(tokens * kv_dim, dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = axk.make_qk_args(tokens=tokens, q_heads=q_heads, k_heads=k_heads, head_dim=D, rope_dim=rope_dim,
                            flags=axk.QK_FLAG_RING | axk.QK_FLAG_CACHE_E4M3, eps=1e-6, mscale=mscale,
                            block_tokens=page_tokens, n_layers=2, layer=0, pool_stride=kv_dim, tbl_stride=pages,
                            n_blocks=pages, q=qd, k=kd, v=vd, q_gamma=qgd, k_gamma=kgd, inv_freq=fd, positions=pd,
                            block_tables=td, k_pool=records.ptr, v_pool=records.ptr + half_bytes, k_out=k_out,
                            status_word=status)
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
    sync()
    assert int(status.item()) == 0 and records.guards_intact()
    got = records.payload().reshape(pages, 2, page_tokens, kv_dim)
    want = np.full_like(got, 0xFF)
    k_rot = k_out.cpu().numpy().view(np.uint16).reshape(tokens, kv_dim)
    for t in range(tokens):
        pos = int(positions[t])
        page, slot = int(table[0, (pos // page_tokens) % pages]), pos % page_tokens
        want[page, 0, slot] = ol.bf16_to_e4m3_scale1(k_rot[t])
        want[page, 1, slot] = ol.bf16_to_e4m3_scale1(v[t].reshape(-1))
    assert np.array_equal(got, want)
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0


def test_streaming_and_per_token_kernels_agree_bitwise(axk, cuda_device):
    """The same 2048 tokens once in one call (streaming kernel) and once in calls of 128 (per-token kernel)."""
    import torch
    from gpu_util import dev, sync

    tokens = 2048
    q, k, v, qg, kg, positions, table = wl.qk_inputs_np(tokens, 64, 8, 128, 4096, seed=11)
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    qgd, kgd, fd, td = dev(qg), dev(kg), dev(inv_freq), dev(table)
    results = []
    for step in (tokens, 128):
        qd, kd, vd, pd = dev(q).view(-1), dev(k).view(-1), dev(v).view(-1), dev(positions)
        kp = torch.full((4096 * 16 * 1024,), -1, dtype=torch.int16, device="cuda")
        vp = torch.full((4096 * 16 * 1024,), -1, dtype=torch.int16, device="cuda")
        ko = torch.zeros(tokens * 1024, dtype=torch.int16, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        for lo in range(0, tokens, step):
            args = axk.make_qk_args(tokens=step, q_heads=64, k_heads=8, head_dim=128, rope_dim=128,
                                    flags=axk.QK_FLAG_RING, eps=1e-6, mscale=mscale, block_tokens=16, n_layers=1,
                                    layer=0, pool_stride=1024, tbl_stride=4096, n_blocks=4096,
                                    q=qd[lo * 8192:], k=kd[lo * 1024:], v=vd[lo * 1024:], q_gamma=qgd, k_gamma=kgd,
                                    inv_freq=fd, positions=pd[lo:], block_tables=td, k_pool=kp, v_pool=vp,
                                    k_out=ko[lo * 1024:], status_word=status)
            assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
        sync()
        assert int(status.item()) == 0
        results.append([x.cpu().numpy() for x in (qd, kp, vp, ko)])
    for a, b in zip(*results):
        assert np.array_equal(a, b)
    assert axk.lib().axiom_b200_pipeline_faults(0) == 0


def test_out_of_range_addresses_raise_status_and_skip(axk, cuda_device):
    """Without ring wrap, positions beyond the table are reported through the status word and not written."""
    import torch
    from gpu_util import Guarded, dev, sync

    tokens, n_blocks = 24, 8
    q, k, v, qg, kg, positions, table = wl.qk_inputs_np(tokens, 4, 2, 128, n_blocks, seed=1, max_base=1)
    positions = (n_blocks * 16 - 8 + np.arange(tokens)).astype(np.uint32)  # the last 16 tokens fall off the table
    table[0, 3] = 99                                                       # and one block id is out of range
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128)
    kv_dim = 256
    pool = Guarded(n_blocks * 16 * kv_dim * 2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qd, kd, qgd, kgd, fd, pd, td = dev(q), dev(k), dev(qg), dev(kg), dev(inv_freq), dev(positions), dev(table)
    args = axk.make_qk_args(tokens=tokens, q_heads=4, k_heads=2, head_dim=128, rope_dim=128, flags=0, eps=1e-6,
                            mscale=1.0, block_tokens=16, n_layers=1, layer=0, pool_stride=kv_dim,
                            tbl_stride=n_blocks, n_blocks=n_blocks, q=qd, k=kd, q_gamma=qgd, k_gamma=kgd,
                            inv_freq=fd, positions=pd, block_tables=td,
                            k_pool=pool.ptr, status_word=status)
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
    sync()
    assert int(status.item()) == axk.STATUS_WORD_BAD_ADDRESS
    assert pool.guards_intact()
    cells = pool.payload(np.uint16).reshape(n_blocks * 16, kv_dim)
    assert int((cells != 0xFFFF).any(axis=1).sum()) == 8  # only the 8 in-range tokens were stored


def test_yarn_table_kernel_matches_oracle(axk, cuda_device):
    import torch
    from gpu_util import sync

    for theta, factor, ctx, dim in [(1e6, 4.0, 32768.0, 128), (1e7, 4.0, 262144.0, 64), (1e4, 1.0, 0.0, 128),
                                    (5e5, 8.0, 8192.0, 256)]:
        out = torch.empty(dim // 2, dtype=torch.float32, device="cuda")
        assert axk.yarn_inv_freq(0, dim, theta, factor, ctx, 32.0, 1.0, out) == axk.AXIOM_OK
        sync()
        got = out.cpu().numpy()
        want = ol.yarn_inv_freq(theta, factor, ctx, 32.0, 1.0, dim) if factor > 1 else \
            np.array([np.float32(theta) ** np.float32(-2.0 * i / dim) for i in range(dim // 2)], np.float32)
        assert np.allclose(got, want, rtol=2e-6, atol=0)
        assert got[0] == 1.0


def test_config3_full_size(axk, cuda_device):
    """Config 3 at its stated size (8192 tokens x (64 q + 8 kv) heads x 128, theta 1e6, YaRN 4 / 32768, 16-token
    pages, seeded permutation of 4096 pages): EVERY token's Q and K output is compared with the CPU oracle under
    the one-BF16-ulp bound of tolerance(), and every K row sits in its page with all other cells untouched."""
    import torch
    from gpu_util import dev, sync

    tokens = 8192
    q, k, v, qg, kg, positions, table = wl.qk_inputs_np(tokens, 64, 8, 128, 4096, seed=3)
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    qd, kd, qgd, kgd, fd, pd, td = dev(q), dev(k), dev(qg), dev(kg), dev(inv_freq), dev(positions), dev(table)
    pool = torch.full((4096 * 16 * 1024,), -1, dtype=torch.int16, device="cuda")
    k_out = torch.full((tokens, 8, 128), -1, dtype=torch.int16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    args = axk.make_qk_args(tokens=tokens, q_heads=64, k_heads=8, head_dim=128, rope_dim=128, flags=axk.QK_FLAG_RING,
                            eps=1e-6, mscale=mscale, block_tokens=16, n_layers=1, layer=0, pool_stride=1024,
                            tbl_stride=4096, n_blocks=4096, q=qd, k=kd, q_gamma=qgd, k_gamma=kgd,
                            inv_freq=fd, positions=pd, block_tables=td, k_pool=pool, k_out=k_out,
                            status_word=status)
    assert axk.qk_norm_rope_paged(0, args) == axk.AXIOM_OK
    sync()
    assert int(status.item()) == 0
    got_q = qd.cpu().numpy().view(np.uint16).reshape(q.shape)
    got_k = k_out.cpu().numpy().view(np.uint16).reshape(k.shape)
    want_q, want_k, want_status = ol.qk_norm_rope_paged(q, k, None, qg, kg, inv_freq, positions, table, rope_dim=128,
                                                        eps=1e-6, mscale=mscale, want_k_out=True)
    assert want_status == 0
    for t0 in range(0, tokens, 1024):  # bounded FP64 temporaries
        sl = slice(t0, t0 + 1024)
        for got, want, src, gamma in ((got_q, want_q, q, qg), (got_k, want_k, k, kg)):
            a, b = wl.from_bf16_bits(got[sl]), wl.from_bf16_bits(want[sl])
            assert np.all(np.abs(a - b) <= tolerance(src[sl], gamma, inv_freq, positions[sl], 128, mscale)), f"tokens {t0}.."
            assert np.mean(got[sl] != want[sl]) < 0.02
    cells = pool.cpu().numpy().view(np.uint16).reshape(4096, 16, 1024)
    lb = (positions // 16) % 4096
    assert np.array_equal(cells[table[0, lb], positions % 16], got_k.reshape(tokens, 1024))
    assert int((cells != 0xFFFF).any(axis=2).sum()) == tokens


def test_round_after_norm_convention_contract(axk, cuda_device):
    """The flag's argument checks and its two cos/sin sources: partial rotation is refused, a table without the flag is
    refused, a position outside the table leaves the token untouched and raises the status word, and without a table
    the factors come from inv_freq and mscale (compared with the CPU restatement fed with the same device-style table)."""
    import torch
    from gpu_util import dev, host, sync

    tokens, heads = 12, 4
    rng = np.random.default_rng(8)
    q = wl.to_bf16_bits(rng.standard_normal((tokens, heads, 128), dtype=np.float32))
    g = wl.to_bf16_bits(1.0 + 0.02 * rng.standard_normal(128, dtype=np.float32))
    inv_freq = ol.yarn_inv_freq(1e6, 4.0, 32768.0, 32.0, 1.0, 128)
    mscale = float(ol.o().axo_yarn_mscale(4.0))
    positions = np.arange(20, 20 + tokens).astype(np.uint32)
    table = ol.rope_table_host(inv_freq, 128, mscale, 28)       # positions 28..31 are outside
    qd, gd, fd, pd, td = dev(q), dev(g), dev(inv_freq), dev(positions), dev(table)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def args(**kw):
        base = dict(tokens=tokens, q_heads=heads, k_heads=0, head_dim=128, rope_dim=128, flags=axk.QK_FLAG_ROUND_AFTER_NORM,
                    eps=1e-6, mscale=mscale, q=qd, q_gamma=gd, inv_freq=fd, positions=pd, status_word=status)
        base.update(kw)
        return axk.make_qk_args(**base)

    inv = axk.AXIOM_ERR_INVALID_ARGUMENT
    assert axk.qk_norm_rope_paged(0, args(rope_dim=64)) == inv
    assert axk.qk_norm_rope_paged(0, args(flags=0, rope_table=td, rope_table_positions=28)) == inv
    assert axk.qk_norm_rope_paged(0, args(rope_table=td, rope_table_positions=0)) == inv
    assert np.array_equal(host(qd, np.uint16).reshape(q.shape), q)   # nothing ran
    # table source, 4 tokens outside
    assert axk.qk_norm_rope_paged(0, args(rope_table=td, rope_table_positions=28)) == axk.AXIOM_OK
    sync()
    got = host(qd, np.uint16).reshape(q.shape)
    want, st = ol.qk_norm_rope_round_after_norm(q, g, table, positions)
    assert st == 1 and int(status.item()) == axk.STATUS_WORD_BAD_ADDRESS
    assert np.array_equal(got[8:], q[8:])
    # three BF16 ulps at the magnitude of the rotation terms: the operands are rounded before the rotation, and the
    # CPU restatement's inverse square root is not the device's
    a, b = wl.from_bf16_bits(got[:8]), wl.from_bf16_bits(want[:8])
    assert np.all(np.abs(a - b) <= 3 * tolerance(q[:8], g, inv_freq, positions[:8], 128, mscale))
    # inv_freq source: same convention, factors evaluated on the device
    qd2 = dev(q)
    status.zero_()
    assert axk.qk_norm_rope_paged(0, args(q=qd2)) == axk.AXIOM_OK
    sync()
    full_table = ol.rope_table_host(inv_freq, 128, mscale, 32)
    want2, _ = ol.qk_norm_rope_round_after_norm(q, g, full_table, positions)
    a, b = wl.from_bf16_bits(host(qd2, np.uint16).reshape(q.shape)), wl.from_bf16_bits(want2)
    assert int(status.item()) == 0
    assert np.all(np.abs(a - b) <= 3 * tolerance(q, g, inv_freq, positions, 128, mscale))
