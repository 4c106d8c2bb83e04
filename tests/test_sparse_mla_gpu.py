"""GPU parity of the sparse MLA decode attention (through the C ABI) against the CPU oracle, which
restates the reference's torch twin (ref_flash_attn over deq_model1_row records) with sums in
double, and against the fixture made with that twin.

Floating point, so a tolerance: the kernel rounds the probabilities to 16 bits before they meet the
values (as the reference kernels do) and its output to bf16.  Per head row the error must stay
below 2^-7 of the row's largest output magnitude, and the cosine against the oracle above 0.9999
(the reference's own end-to-end gate for this stage is cosine > 0.98)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu

SCALE = 512 ** -0.5


def u16(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def from_u16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).cuda()


def model1_pool(rng, pages, epb, exp_lo=115, exp_hi=122):
    """Random MODEL1 records: finite e4m3 bytes, scale exponents in [exp_lo, exp_hi), bf16 rotary values."""
    stride = -(-epb * 584 // 576) * 576
    pool = np.zeros((pages, stride), np.uint8)
    body = rng.integers(0, 256, (pages, epb, 448)).astype(np.uint8)
    body = np.where((body & 0x7f) == 0x7f, body & 0x80, body).astype(np.uint8)
    rope = oracle.f32_to_bf16((rng.standard_normal((pages, epb, 64)) * 0.7).astype(np.float32)).view(np.uint8)
    pool[:, :epb * 576] = np.concatenate([body, rope.reshape(pages, epb, 128)], axis=-1).reshape(pages, epb * 576)
    sb = np.zeros((pages, epb, 8), np.uint8)
    sb[..., :7] = rng.integers(exp_lo, exp_hi, (pages, epb, 7))
    pool[:, epb * 576:epb * 584] = sb.reshape(pages, epb * 8)
    return pool


def view4(pool, epb):
    """The [pages, entries, 1, 584] view the cache manager hands to the attention."""
    t = torch.from_numpy(pool).cuda()
    return t.as_strided((t.size(0), epb, 1, 584), (t.size(1), 584, 584, 1))


def indices(rng, batch, cap, lens, entries, holes=0):
    idx = np.full((batch, cap), -1, np.int32)
    for b in range(batch):
        idx[b, :lens[b]] = rng.choice(entries, size=lens[b], replace=lens[b] > entries)
        if holes and lens[b] > 2:
            idx[b, rng.choice(lens[b], size=min(holes, lens[b] - 1), replace=False)] = -1
    return idx


def check_close(got_u16, ref):
    got = oracle.bf16_to_f32(got_u16).astype(np.float64)
    ref = ref.astype(np.float64)
    row_max = np.abs(ref).max(axis=-1, keepdims=True)
    assert np.all(np.abs(got - ref) <= row_max * 2.0 ** -7 + 1e-6), float(np.max(np.abs(got - ref) / (row_max + 1e-30)))
    dot = (got * ref).sum(-1)
    norm = np.sqrt((got * got).sum(-1) * (ref * ref).sum(-1))
    live = norm > 0
    assert np.all(dot[live] / norm[live] > 0.9999)
    assert np.all(got[~live] == 0)


def run(wuda, q, swa, cmp, sink, scale=SCALE, split=True):
    """swa / cmp = None or (pool, epb, idx, lens) in numpy; q uint16 [batch, heads, 512]."""
    status = wuda.device_status_word()
    status.zero_()
    args = []
    for t in (swa, cmp):
        if t is None:
            args += [None, None, None]
        else:
            args += [view4(t[0], t[1]), torch.from_numpy(t[2]).cuda(), torch.from_numpy(np.asarray(t[3], np.int32)).cuda()]
    out = wuda.sparse_mla_decode(from_u16(q), *args, None if sink is None else torch.from_numpy(sink).cuda(), scale,
                                 status_word=status, split=split)
    torch.cuda.synchronize()
    return u16(out), int(status.item())


def test_golden(wuda):
    g = load_golden("sparse_mla_h16.npz")
    got, status = run(wuda, g["q"], (g["swa_pool"], int(g["swa_epb"]), g["swa_idx"], g["swa_len"]),
                      (g["cmp_pool"], int(g["cmp_epb"]), g["cmp_idx"], g["cmp_len"]), g["sink"], float(g["scale"]))
    assert status == 0
    check_close(got, g["out"])


@pytest.mark.parametrize("batch,heads,swa_lens,cmp_lens,holes,with_sink,q_gain", [
    (2, 128, [128, 128], [2048, 1500], 0, True, 1.0),     # the full window and top-k of a long context
    (3, 64, [17, 128, 1], [100, 0, 31], 3, True, 1.0),    # ragged, skipped entries, one pool empty for a request
    (1, 128, [0], [5], 0, False, 1.0),                    # fewer keys than one block, no sink
    (2, 8, [33, 64], None, 0, True, 1.0),                 # window pool only
    (2, 16, None, [300, 64], 2, False, 1.0),              # top-k pool only
    (2, 128, [128, 40], [1024, 700], 0, True, 8.0),       # peaked softmax: the running maximum grows often
    (4, 128, [0, 5, 0, 128], [0, 0, 0, 2048], 0, True, 1.0),   # requests without any key give zero rows
])
@pytest.mark.parametrize("split", [False, True])   # one CTA per request and half / several with a merge launch
def test_against_oracle(wuda, batch, heads, swa_lens, cmp_lens, holes, with_sink, q_gain, split):
    rng = np.random.default_rng(batch * 1009 + heads * 31 + int(q_gain))
    swa = cmp = None
    if swa_lens is not None:
        pool = model1_pool(rng, 3, 256)
        swa = (pool, 256, indices(rng, batch, 128, swa_lens, 3 * 256, holes), swa_lens)
    if cmp_lens is not None:
        pool = model1_pool(rng, 40, 64)
        cmp = (pool, 64, indices(rng, batch, 2048, cmp_lens, 40 * 64, holes), cmp_lens)
    q = oracle.f32_to_bf16((rng.standard_normal((batch, heads, 512)) * q_gain).astype(np.float32))
    sink = rng.standard_normal(heads).astype(np.float32) if with_sink else None
    got, status = run(wuda, q, swa, cmp, sink, split=split)
    assert status == 0
    check_close(got, oracle.sparse_mla(q, swa, cmp, sink, SCALE))


def test_rising_logits_rescale_the_accumulator(wuda):
    """Keys ordered so that every block's largest logit exceeds the one before by more than the lazy
    threshold: the accumulator in tensor memory is rescaled block after block."""
    rng = np.random.default_rng(5)
    pool = model1_pool(rng, 8, 64)
    n = 320
    q = oracle.f32_to_bf16((rng.standard_normal((1, 128, 512)) * 3).astype(np.float32))
    # order the keys by their logit for head 0, so that this head's maximum keeps growing
    qf = oracle.bf16_to_f32(q[0, 0]).astype(np.float64)
    logits = []
    for t in range(n):
        one = oracle.sparse_mla(q[:, :1], None, (pool, 64, np.array([[t]], np.int32), [1]), None, SCALE)[0, 0]
        logits.append(float(qf @ one.astype(np.float64)))   # one key: the output is the key itself
    order = np.argsort(np.asarray(logits)).astype(np.int32)[None, :]
    ref = oracle.sparse_mla(q, None, (pool, 64, order, [n]), None, SCALE)
    for split in (False, True):
        got, status = run(wuda, q, None, (pool, 64, order, [n]), None, split=split)
        assert status == 0
        check_close(got, ref)


def test_reference_call_form(wuda):
    """The keyword form of the layer step's call: [batch, 1, heads, 512] query, [batch, 1, topk] indices."""
    rng = np.random.default_rng(77)
    batch, heads = 2, 128
    swa_pool, cmp_pool = model1_pool(rng, 2, 256), model1_pool(rng, 10, 64)
    swa_lens, cmp_lens = [128, 90], [512, 333]
    swa_idx, cmp_idx = indices(rng, batch, 128, swa_lens, 512), indices(rng, batch, 512, cmp_lens, 640)
    q = oracle.f32_to_bf16(rng.standard_normal((batch, heads, 512)).astype(np.float32))
    sink = rng.standard_normal(heads).astype(np.float32)
    out, lse = wuda.flash_mla_with_kvcache(
        q=from_u16(q).view(batch, 1, heads, 512), k_cache=view4(swa_pool, 256), block_table=None, cache_seqlens=None,
        head_dim_v=512, tile_scheduler_metadata=None, num_splits=None, softmax_scale=SCALE, causal=False,
        is_fp8_kvcache=True, indices=torch.from_numpy(swa_idx).cuda().view(batch, 1, 128),
        topk_length=torch.tensor(swa_lens, dtype=torch.int32).cuda(), extra_k_cache=view4(cmp_pool, 64),
        extra_indices_in_kvcache=torch.from_numpy(cmp_idx).cuda().view(batch, 1, 512),
        extra_topk_length=torch.tensor(cmp_lens, dtype=torch.int32).cuda(), attn_sink=torch.from_numpy(sink).cuda())
    torch.cuda.synchronize()
    assert lse is None and tuple(out.shape) == (batch, 1, heads, 512)
    ref = oracle.sparse_mla(q, (swa_pool, 256, swa_idx, swa_lens), (cmp_pool, 64, cmp_idx, cmp_lens), sink, SCALE)
    check_close(u16(out).reshape(batch, heads, 512), ref)


def test_index_outside_the_pool_is_skipped_and_reported(wuda):
    rng = np.random.default_rng(9)
    pool = model1_pool(rng, 2, 64)
    idx = indices(rng, 1, 64, [40], 128)
    bad = idx.copy()
    bad[0, 7] = 128 + 5          # one past the last page
    q = oracle.f32_to_bf16(rng.standard_normal((1, 32, 512)).astype(np.float32))
    got, status = run(wuda, q, None, (pool, 64, bad, [40]), None)
    assert status == 110   # WUDA_DEV_BAD_PAGE_INDEX
    skipped = idx.copy()
    skipped[0, 7] = -1
    check_close(got, oracle.sparse_mla(q, None, (pool, 64, skipped, [40]), None, SCALE))


def test_scale_exponent_outside_the_exact_range_is_clamped_and_reported(wuda):
    """Key values are exact for scale exponents in [-15, 7]; a byte beyond that is clamped and reported."""
    rng = np.random.default_rng(13)
    pool = model1_pool(rng, 1, 64)
    idx = np.arange(40, dtype=np.int32)[None, :]
    q = oracle.f32_to_bf16(rng.standard_normal((1, 16, 512)).astype(np.float32))
    edge = pool.copy()
    edge[0, 64 * 576 + 3 * 8 + 2] = 127 - 15     # the lower edge of the range: still exact
    edge[0, 64 * 576 + 5 * 8 + 0] = 127 + 7      # the upper edge
    got, status = run(wuda, q, None, (edge, 64, idx, [40]), None)
    assert status == 0
    check_close(got, oracle.sparse_mla(q, None, (edge, 64, idx, [40]), None, SCALE))
    beyond = pool.copy()
    beyond[0, 64 * 576 + 3 * 8 + 2] = 127 + 9
    got, status = run(wuda, q, None, (beyond, 64, idx, [40]), None)
    assert status == 156   # WUDA_DEV_MLA_SCALE_RANGE
    clamped = pool.copy()
    clamped[0, 64 * 576 + 3 * 8 + 2] = 127 + 7
    check_close(got, oracle.sparse_mla(q, None, (clamped, 64, idx, [40]), None, SCALE))


def test_argument_checks(wuda):
    from wuda_b200._lib import WudaError
    rng = np.random.default_rng(1)
    pool = view4(model1_pool(rng, 1, 64), 64)
    q = torch.zeros(1, 129, 512, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(1, 8, dtype=torch.int32, device="cuda")
    lens = torch.ones(1, dtype=torch.int32, device="cuda")
    with pytest.raises(WudaError):
        wuda.sparse_mla_decode(q, pool, idx, lens)            # more than 128 heads
    with pytest.raises(WudaError):
        wuda.sparse_mla_decode(q[:, :64].contiguous(), pool, idx, lens, softmax_scale=-1.0)
