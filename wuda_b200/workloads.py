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
