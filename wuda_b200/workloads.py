"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations.  Everything is generated on the host (numpy / torch CPU) so the CPU
oracle and the GPU kernels consume identical bytes.
"""
import numpy as np
import torch

HEADS, DIM = 64, 128


def _e4m3_bytes(t):
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def make_mqa_case(batch, next_n, ctx_lo, ctx_hi, epb=64, seed=0xB200, spare_pages=3, page_pad=0,
                  ctx=None, shuffle=True):
    """Paged MQA-logits inputs.

    q ~ N(0,1) clipped to +-448 -> e4m3 [batch*next_n, 64, 128]; request b has ctx_b ~
    U{ctx_lo..ctx_hi} tokens (or `ctx[b]`), its row j sees ctx_b - next_n + 1 + j of
    them; keys ~ N(0,1) -> e4m3 in pages of `epb` tokens followed by epb fp32 per-token
    scales ~ U(0.01, 0.1); the block table is one seeded permutation of the physical
    pages (plus `spare_pages` unused pages; padding and spare pages hold 0xA5); head
    weights ~ N(0, 1/64).  Unused block-table entries are -1.
    Returns a dict of numpy arrays.
    """
    rng = np.random.default_rng(seed)
    g = torch.Generator().manual_seed(int(seed))
    rows = batch * next_n
    if ctx is None:
        ctx = rng.integers(ctx_lo, ctx_hi + 1, size=batch)
    ctx = np.asarray(ctx, dtype=np.int64)
    context_lens = np.maximum(ctx[:, None] - next_n + 1 + np.arange(next_n)[None, :], 0).astype(np.int32)
    pages = (ctx + epb - 1) // epb
    total_pages = int(pages.sum())
    num_blocks = max(total_pages + spare_pages, 1)
    perm = rng.permutation(num_blocks) if shuffle else np.arange(num_blocks)
    max_pages = max(int(pages.max()) if batch else 1, 1)
    block_table = np.full((batch, max_pages), -1, np.int32)
    off = 0
    for b in range(batch):
        block_table[b, :pages[b]] = perm[off:off + pages[b]]
        off += pages[b]
    used = perm[:total_pages]
    payload = epb * (DIM + 4)
    stride = payload + page_pad
    assert stride % 16 == 0
    kv_pages = np.full((num_blocks, stride), 0xA5, np.uint8)
    # keys, generated in chunks to bound host memory
    chunk = 4096
    for s in range(0, total_pages, chunk):
        e = min(total_pages, s + chunk)
        k = torch.randn((e - s) * epb, DIM, generator=g)
        kv_pages[used[s:e], :epb * DIM] = _e4m3_bytes(k).reshape(e - s, epb * DIM)
        sc = (torch.rand((e - s) * epb, generator=g) * 0.09 + 0.01).numpy().astype(np.float32)
        kv_pages[used[s:e], epb * DIM:payload] = sc.view(np.uint8).reshape(e - s, epb * 4)
    q = _e4m3_bytes(torch.randn(rows, HEADS, DIM, generator=g).clamp_(-448, 448))
    weights = (torch.randn(rows, HEADS, generator=g) / 8.0).numpy().astype(np.float32)
    max_ctx = int(ctx.max()) if batch else 0
    return dict(q=q, kv_pages=kv_pages, weights=weights, context_lens=context_lens, block_table=block_table,
                ctx=ctx, batch=batch, next_n=next_n, epb=epb, num_blocks=num_blocks, page_stride=stride,
                logits_stride=max((max_ctx + 255) // 256 * 256, 256))


def mqa_algorithmic_bytes(case):
    """Bytes one launch must move (DESIGN: KV read once per request, fp32 logits out,
    q + weights in): sum_b ctx_b*132 + sum_rows ctx*4 + rows*(64*128 + 64*4)."""
    rows = case["batch"] * case["next_n"]
    return int(case["ctx"].sum()) * 132 + int(case["context_lens"].sum()) * 4 + rows * (HEADS * DIM + HEADS * 4)


def to_device(case, device="cuda"):
    """Upload the arrays of a case; q becomes a float8_e4m3fn tensor."""
    out = dict(case)
    out["q"] = torch.from_numpy(case["q"]).to(device).view(torch.float8_e4m3fn)
    for k in ("kv_pages", "weights", "context_lens", "block_table"):
        out[k] = torch.from_numpy(case[k]).to(device)
    return out


def quantize_fp8_1x128(x):
    """fp32 [M, K] -> (e4m3 bytes [M, K], fp32 scales [M, K/128]); scale = max(amax, 1e-4) / 448
    (origin/kernel.py:79-83)."""
    m, k = x.shape
    v = torch.as_tensor(x, dtype=torch.float32).view(m, k // 128, 128)
    s = v.abs().amax(-1).clamp_min(1e-4) * (1.0 / 448.0)
    q = (v / s.unsqueeze(-1)).clamp(-448, 448).view(m, k)
    return _e4m3_bytes(q), s.numpy().astype(np.float32)


def quantize_fp8_128x128(w):
    """fp32 [N, K] -> (e4m3 bytes [N, K], fp32 scales [ceil(N/128), K/128])."""
    n, k = w.shape
    nt = (n + 127) // 128
    wp = torch.zeros(nt * 128, k)
    wp[:n] = torch.as_tensor(w, dtype=torch.float32)
    v = wp.view(nt, 128, k // 128, 128)
    s = v.abs().amax(dim=(1, 3)).clamp_min(1e-4) * (1.0 / 448.0)
    q = (v / s[:, None, :, None]).clamp(-448, 448).view(nt * 128, k)[:n]
    return _e4m3_bytes(q.contiguous()), s.numpy().astype(np.float32)


def make_gemm_fp8_case(m, n, k, seed=0xB202):
    """Activations ~ N(0,1), weights ~ N(0, 0.02), quantised to e4m3 with 1x128 / 128x128 fp32 scales."""
    g = torch.Generator().manual_seed(int(seed))
    a, a_s = quantize_fp8_1x128(torch.randn(m, k, generator=g))
    w, w_s = quantize_fp8_128x128(torch.randn(n, k, generator=g) * 0.02)
    return dict(a=a, a_s=a_s, w=w, w_s=w_s, m=m, n=n, k=k)


def gemm_fp8_algorithmic_bytes(m, n, k):
    """N*K weights + their scales + M*K activations + their scales + M*N bf16 output."""
    return n * k + ((n + 127) // 128) * (k // 128) * 4 + m * k + m * (k // 128) * 4 + m * n * 2


E2M1_BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def quantize_nvfp4(x):
    """fp32 [R, K] -> (packed e2m1 uint8 [R, K/2], ue4m3 scale bytes [R, K/16], per-tensor fp32 scale).
    x ~= e2m1 * ue4m3(scale of its 16-element block) * tensor scale, tensor scale = amax / (448 * 6)."""
    x = torch.as_tensor(x, dtype=torch.float32)
    r, k = x.shape
    amax = float(x.abs().max())
    gs = amax / (448.0 * 6.0) if amax > 0 else 1.0
    v = x.view(r, k // 16, 16)
    sf = (v.abs().amax(-1) / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    sf_dec = sf.float()
    scaled = torch.where(sf_dec.unsqueeze(-1) > 0, v / (sf_dec.unsqueeze(-1) * gs), torch.zeros_like(v))
    ax = scaled.abs().clamp_max(6.0)
    idx = torch.bucketize(ax, E2M1_BOUNDS)                     # ties go to the smaller magnitude
    code = idx.to(torch.uint8) | (((scaled < 0) & (idx != 0)).to(torch.uint8) << 3)
    code = code.view(r, k // 2, 2)
    packed = (code[:, :, 0] & 15) | (code[:, :, 1] << 4)
    return packed.contiguous().numpy(), sf.view(torch.uint8).numpy().copy(), np.float32(gs)


def pack_nvfp4_scales(sf, rows_pad=128):
    """Scale bytes [R, K/16] -> the layout the tensor core's scale copy expects, per 128 rows x 256 K:
    [row tile][K/256][4 (K/64 step)][32 (row % 32)][4 (row / 32)][4 (scale within the step)] bytes."""
    r, g = sf.shape
    assert g % 16 == 0
    rt = (r + rows_pad - 1) // rows_pad
    buf = np.zeros((rt * rows_pad, g), np.uint8)
    buf[:r] = sf
    v = buf.reshape(rt, 4, 32, g // 16, 4, 4)          # [tile][row/32][row%32][kb][step][byte]
    return np.ascontiguousarray(v.transpose(0, 3, 4, 2, 1, 5)).reshape(-1)


def make_gemm_nvfp4_case(m, n, k, seed=0xB203):
    g = torch.Generator().manual_seed(int(seed))
    a, a_sf, a_gs = quantize_nvfp4(torch.randn(m, k, generator=g))
    w, w_sf, w_gs = quantize_nvfp4(torch.randn(n, k, generator=g) * 0.02)
    return dict(a=a, a_sf=a_sf, a_gs=a_gs, w=w, w_sf=w_sf, w_gs=w_gs, m=m, n=n, k=k,
                a_sf_packed=pack_nvfp4_scales(a_sf), w_sf_packed=pack_nvfp4_scales(w_sf))


def gemm_nvfp4_algorithmic_bytes(m, n, k):
    return n * k // 2 + n * k // 16 + 4 + m * k // 2 + m * k // 16 + 4 + m * n * 2
