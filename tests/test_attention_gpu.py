"""Attention-forward parity: the sm_100a kernel through the C ABI against the composed CPU
oracle (no reference vector exists for attention: parity unpinned, see oracle/sile_oracle.h).

Tolerance: max-abs error <= 2e-2 of the output scale (bf16 in/out, f32 accumulation)."""
import numpy as np
import pytest

from _util import rel_err

pytestmark = pytest.mark.gpu
BF16_TOL = 2e-2


@pytest.fixture(scope="module")
def sb():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sile_b200
    return sile_b200


@pytest.fixture(params=["single", "split", "persistent", "pair"], autouse=True)
def attn_kernel(request, monkeypatch):
    """Every case runs on all four kernels: the one-CTA-per-item kernel, the same with every
    tile's softmax spread over eight warps, the persistent kernel and the CTA-pair
    (cta_group::2) one."""
    monkeypatch.setenv("SILE_CUDA_ATTN_KERNEL", request.param)
    return request.param


def _inputs(bh, s, d, seed):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn(bh, s, d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
            for _ in range(3)]


def _oracle_units(oracle, q, k, v, heads, s, d, scale, causal, units_per_head, bm=128):
    """Runs the oracle on the listed heads; returns {(head, q_tile): [bm, d] rows}."""
    out = {}
    for h in heads:
        qh = q[h].float().cpu().numpy().reshape(s, d)
        kt = np.ascontiguousarray(k[h].float().cpu().numpy().reshape(s, d).T)
        vh = v[h].float().cpu().numpy().reshape(s, d)
        tiles = units_per_head[h] if units_per_head is not None else None
        o = oracle.attention(qh, kt, vh, 1, s, d, bm, 64, scale, causal, tiles)
        for t in (tiles if tiles is not None else range(s // bm)):
            out[(h, int(t))] = o[t * bm:(t + 1) * bm]
    return out


@pytest.mark.parametrize("bh,s", [(2, 256), (3, 384), (1, 128), (2, 1024)])
@pytest.mark.parametrize("causal", [False, True])
def test_small_full(sb, oracle, bh, s, causal):
    import torch
    d, scale = 128, 1.0 / np.sqrt(128)
    q, k, v = _inputs(bh, s, d, 100 + s)
    o = torch.zeros_like(q)
    sb.attention(q, k, v, o, scale, causal).apply()
    sb.synchronize()
    kt = np.ascontiguousarray(k.float().cpu().numpy().transpose(0, 2, 1)).reshape(bh * d, s)
    want = oracle.attention(q.float().cpu().numpy().reshape(bh * s, d), kt,
                            v.float().cpu().numpy().reshape(bh * s, d), bh, s, d, 64, 64, scale, causal)
    assert rel_err(o.float().cpu().numpy().reshape(bh * s, d), want) < BF16_TOL


def _largest_divisor(n, limit=64):
    return max(x for x in range(1, min(n, limit) + 1) if n % x == 0)


def _oracle_full(oracle, q, k, v, scale, causal):
    """The composed oracle on whole [bh, s, d] tensors, with logical tiles that divide s."""
    bh, s, d = q.shape
    t = _largest_divisor(s)
    kt = np.ascontiguousarray(k.float().cpu().numpy().transpose(0, 2, 1)).reshape(bh * d, s)
    return oracle.attention(q.float().cpu().numpy().reshape(bh * s, d), kt, v.float().cpu().numpy().reshape(bh * s, d),
                            bh, s, d, t, t, scale, causal).reshape(bh, s, d)


@pytest.mark.parametrize("s", [1, 100, 200, 333, 1000])
@pytest.mark.parametrize("causal", [False, True])
def test_ragged_sequence(sb, oracle, causal, s):
    # lengths that are not multiples of the key block / query tile: against the oracle (run with
    # logical tiles that divide the length) and against float64
    import torch
    bh, d, scale = 2, 128, 0.11
    q, k, v = _inputs(bh, s, d, 7 + s)
    o = torch.full_like(q, 3.0)
    sb.attention(q, k, v, o, scale, causal).apply()
    sb.synchronize()
    assert rel_err(o.float().cpu().numpy(), _oracle_full(oracle, q, k, v, scale, causal)) < BF16_TOL
    sc = torch.einsum("bqd,bkd->bqk", q.double(), k.double()) * scale
    if causal:
        sc = sc.masked_fill(~torch.tril(torch.ones(s, s, dtype=torch.bool, device="cuda")), float("-inf"))
    want = torch.einsum("bqk,bkd->bqd", torch.softmax(sc, -1), v.double())
    assert rel_err(o.double().cpu().numpy(), want.cpu().numpy()) < BF16_TOL


def test_rank4_shapes_and_rows_sum_to_one(sb):
    # V = 1 makes every output element the softmax row sum
    import torch
    q, k, _ = _inputs(8, 512, 128, 5)
    q, k = q.view(2, 4, 512, 128), k.view(2, 4, 512, 128)
    v = torch.ones_like(q)
    o = torch.zeros_like(q)
    sb.attention(q, k, v, o, 0.3, True).apply()
    sb.synchronize()
    assert (o.float() - 1.0).abs().max().item() < 1e-2


def test_large_logits_and_rescale_path(sb, oracle):
    # scores whose row max keeps growing by more than the lazy-rescale threshold
    import torch
    bh, s, d = 1, 1024, 128
    q, k, v = _inputs(bh, s, d, 11)
    ramp = torch.linspace(0.0, 6.0, s, device="cuda").view(1, s, 1)
    k = (k.float() * 0.2 + ramp * q.float().mean(dim=1, keepdim=True).sign()).to(torch.bfloat16)
    o = torch.zeros_like(q)
    sb.attention(q, k, v, o, 1.0, False).apply()
    sb.synchronize()
    assert rel_err(o.float().cpu().numpy(), _oracle_full(oracle, q, k, v, 1.0, False)) < BF16_TOL
    sc = torch.einsum("bqd,bkd->bqk", q.double(), k.double())
    want = torch.einsum("bqk,bkd->bqd", torch.softmax(sc, -1), v.double())
    assert rel_err(o.double().cpu().numpy(), want.cpu().numpy()) < BF16_TOL


@pytest.mark.parametrize("step", [9.0, 20.0])
def test_row_max_crosses_the_rescale_threshold_many_times_under_a_causal_mask(sb, oracle, step):
    """Keys whose scores climb by `step` (log2 units, beyond the 2^8 lazy-rescale threshold) from
    one 128-key block to the next: every later query row sees its running max jump at every block
    it may attend to, so the accumulator is rescaled once per block, the diagonal block included."""
    import torch
    bh, s, d = 2, 1536, 128
    g = torch.Generator(device="cuda").manual_seed(31)
    q = torch.ones(bh, s, d, device="cuda") + 0.05 * torch.randn(bh, s, d, generator=g, device="cuda")
    blocks = torch.arange(s, device="cuda") // 128
    # q . k = 128 * level / 128 * (1 + noise); with scale = ln 2 one level is one log2 unit
    level = (blocks.float() * step).view(1, s, 1)
    k = (level / d) * torch.ones(bh, s, d, device="cuda") + 0.02 * torch.randn(bh, s, d, generator=g, device="cuda")
    v = torch.randn(bh, s, d, generator=g, device="cuda")
    q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    o = torch.zeros_like(q)
    scale = float(np.log(2.0))
    sb.attention(q, k, v, o, scale, True).apply()
    sb.synchronize()
    assert rel_err(o.float().cpu().numpy(), _oracle_full(oracle, q, k, v, scale, True)) < BF16_TOL


def test_rejects_unsupported(sb):
    import torch
    q = torch.zeros(2, 128, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(sb.SileError) as e:
        sb.attention(q, q, q, torch.zeros_like(q), 1.0).apply()
    assert e.value.code == sb._lib.ERR_UNSUPPORTED
    q = torch.zeros(2, 128, 128, device="cuda", dtype=torch.float32)
    with pytest.raises(sb.SileError):
        sb.attention(q, q, q, torch.zeros_like(q), 1.0).apply()


def _sampled_config(sb, oracle, b, h, s, causal, seed, extra_heads=()):
    import torch
    d, scale = 128, 1.0 / np.sqrt(128)
    bh = b * h
    q, k, v = _inputs(bh, s, d, seed)
    o = torch.zeros_like(q)
    sb.attention(q.view(b, h, s, d), k.view(b, h, s, d), v.view(b, h, s, d), o.view(b, h, s, d), scale, causal).apply()
    sb.synchronize()
    rng = np.random.default_rng(0)
    heads = sorted(set(int(x) for x in rng.choice(bh, size=4, replace=False)) | set(extra_heads))
    n_tiles = s // 128
    units = {hd: sorted(set([n_tiles - 1] + [int(x) for x in rng.choice(n_tiles, size=2, replace=False)])) for hd in heads}
    want = _oracle_units(oracle, q, k, v, heads, s, d, scale, causal, units)
    worst = 0.0
    for (hd, t), rows in want.items():
        got = o[hd, t * 128:(t + 1) * 128].float().cpu().numpy()
        worst = max(worst, rel_err(got, rows))
    assert worst < BF16_TOL
    # linearity in V at full size: O(2V) == 2 O(V) exactly (power-of-two scaling commutes with rounding)
    o2 = torch.zeros_like(q)
    sb.attention(q, k, (v * 2).contiguous(), o2, scale, causal).apply()
    sb.synchronize()
    assert torch.equal(o2, o * 2)


def test_a4_noncausal_b4_h32_s4096_sampled(sb, oracle):
    _sampled_config(sb, oracle, 4, 32, 4096, False, 0)


def test_a5_causal_shard_h32_s8192_sampled(sb, oracle):
    # one GPU's shard of the batch 8 x 32 heads configuration: 32 (batch, head) pairs
    _sampled_config(sb, oracle, 1, 32, 8192, True, 1)


def test_a5_full_causal_b8_h32_s8192_sampled(sb, oracle, attn_kernel):
    """The whole second attention configuration on one GPU: 256 (batch, head) pairs of 8192 causal
    queries.  Sampled (head, q-tile) units -- first and last head, the last q tile included --
    against the oracle, and linearity in V at full size."""
    if attn_kernel == "pair":
        pytest.skip("2 GiB of inputs three times over: the two single-CTA kernels cover the configuration")
    _sampled_config(sb, oracle, 8, 32, 8192, True, 2, extra_heads=(0, 255))


def test_exact_abi_f32_attention(sb, oracle, attn_kernel):
    """sile_kernel_attention: host f32 buffers in the reference's rank-2 layout, K transposed, tile
    sizes / causal / scale bound beforehand; a short grid leaves the query tiles past it untouched.
    Inputs are rounded to bf16 on the device, hence the 16-bit tolerance."""
    bh, s, d, bm, bn = 3, 384, 128, 64, 32
    rng = np.random.default_rng(5)
    q = rng.standard_normal((bh * s, d), dtype=np.float32)
    k = rng.standard_normal((bh, s, d), dtype=np.float32)
    v = rng.standard_normal((bh * s, d), dtype=np.float32)
    kt = np.ascontiguousarray(k.transpose(0, 2, 1)).reshape(bh * d, s)
    scale = float(1.0 / np.sqrt(d))
    for causal in (False, True):
        sb.bind_consts("attention", (bm, bn, int(causal)))
        sb.bind_scale("attention", scale)
        o = np.full((bh * s, d), -7.0, np.float32)
        ntiles = bh * s // bm - 5
        sb.kernel_call("attention", [q, kt, v, o], grid=(ntiles, 1, 1))
        want = oracle.attention(q, kt, v, bh, s, d, bm, bn, scale, causal, units=np.arange(ntiles))
        assert (o[ntiles * bm:] == -7.0).all()
        assert rel_err(o[:ntiles * bm], want[:ntiles * bm]) < BF16_TOL
    # a query tile that would straddle two heads, or keys the composed loop would drop: refused
    sb.bind_consts("attention", (256, 32, 0))
    with pytest.raises(sb.SileError) as e:
        sb.kernel_call("attention", [q, kt, v, np.zeros_like(q)], grid=(1, 1, 1))
    assert e.value.code == sb._lib.ERR_UNSUPPORTED


def test_f32_attention_on_device_buffers(sb, oracle, attn_kernel):
    import torch
    bh, s, d, bm, bn = 2, 256, 128, 128, 64
    rng = np.random.default_rng(9)
    q = rng.standard_normal((bh * s, d), dtype=np.float32)
    kt = rng.standard_normal((bh * d, s), dtype=np.float32)
    v = rng.standard_normal((bh * s, d), dtype=np.float32)
    do = torch.zeros(bh * s, d, device="cuda")
    sb.attention_f32(torch.from_numpy(q).cuda(), torch.from_numpy(kt).cuda(), torch.from_numpy(v).cuda(), do, bm, bn, 0.1, True).apply()
    sb.synchronize()
    want = oracle.attention(q, kt, v, bh, s, d, bm, bn, 0.1, True)
    assert rel_err(do.cpu().numpy(), want) < BF16_TOL


@pytest.mark.parametrize("causal", [False, True])
def test_fused_allgather_epilogue_on_one_gpu(sb, attn_kernel, causal):
    """sile_cuda_attention_allgather with the ranks played in turn on one GPU: every "rank" owns a
    slab of heads and stores it into all destination buffers; afterwards each buffer must equal
    the unsharded result."""
    import torch
    if attn_kernel == "pair":
        pytest.skip("the entry point runs the persistent or the one-CTA-per-item kernel only")
    world, bh_local, s = 4, 3, 700
    q, k, v = _inputs(world * bh_local, s, 128, 21)
    want = torch.zeros_like(q)
    sb.attention(q, k, v, want, 0.09, causal).apply()
    bufs = [torch.full_like(q, 5.0) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(world):
        sl = slice(r * bh_local, (r + 1) * bh_local)
        sb.attention_allgather(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), ptrs, r, 0.09, causal)
    sb.synchronize()
    for b in bufs:
        assert torch.equal(b, want)


@pytest.mark.parametrize("causal", [False, True])
def test_host_buffer_launch_pipelines_head_chunks_and_matches_device_launch(sb, attn_kernel, causal):
    """sile_cuda_launch_host streams a many-head attention in chunks of heads (copies in, kernels
    and copies out overlapped); the result must equal the device-resident launch bit for bit.
    72 heads x 3968 x 128: nine chunks of eight heads, the sequence not a multiple of the block."""
    import torch
    if attn_kernel != "single":
        pytest.skip("one kernel is enough for the host pipeline")
    bh, s = 72, 3968
    g = torch.Generator().manual_seed(5)
    q, k, v = [torch.randn(bh, s, 128, generator=g).to(torch.bfloat16).pin_memory() for _ in range(3)]
    o_host = torch.zeros(bh, s, 128, dtype=torch.bfloat16).pin_memory()
    if causal:   # the same buffers described as rank 4, [batch, heads, S, D]
        sb.attention(q.view(2, 36, s, 128), k.view(2, 36, s, 128), v.view(2, 36, s, 128), o_host.view(2, 36, s, 128), 0.088, causal).apply_host()
    else:
        sb.attention(q, k, v, o_host, 0.088, causal).apply_host()
    o_dev = torch.zeros(bh, s, 128, device="cuda", dtype=torch.bfloat16)
    sb.attention(q.cuda(), k.cuda(), v.cuda(), o_dev, 0.088, causal).apply()
    sb.synchronize()
    assert torch.equal(o_host, o_dev.cpu())
