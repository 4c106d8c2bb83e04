"""Host-side allocation and addressing of the decode caches.

Mirrors the interface of the reference's KVCacheManager
(dsv4_megakernel/megakernel/test/kv_cache_manager.py:53-257): two fp32 state rings and
three paged byte pools whose contents are written by kernels; this class only hands out
slots and pages and computes the rows and destination entries of a decode step.

Layouts (same file, :13-19, :28-50):
  main_state fp32 [capacity, ring, 2048] = [kv 1024 | score 1024], reset to 0 / -inf
  idx_state  fp32 [capacity, ring,  512] = [kv  256 | score  256]
  swa pool  : 584-byte MODEL1 records, 256 per page   (sliding window, ring of 128 tokens)
  cmp pool  : 584-byte MODEL1 records,  64 per page   (one entry per 4 tokens)
  idx pool  : 132-byte FP8 indexer records (128 key bytes + fp32 scale), 64 per page,
              a page holds all key bytes first, then all scales — the page format
              wuda_mqa_logits_fp8 reads
  a destination is page * entries_per_block + offset; -1 means "no write this step".
Page strides of the MODEL1 pools are rounded up to a multiple of 576 bytes.
"""
import numpy as np
import torch

TOKENS_PER_BLOCK = 256
RATIO = 4                 # tokens per compressed entry
WIN = 128                 # sliding-window ring
MIN_RING = 8              # the compressor's overlap window
M1_BODY, M1_RECORD = 576, 584          # 448 fp8 + 64 bf16 rope dims, + 7 scale bytes + 1 pad
IDX_DIM = 128
NEG_INF = float("-inf")


def _round_up(v, a):
    return (v + a - 1) // a * a


class _PagePool:
    """A byte pool of fixed-size pages with a free stack (lowest page first)."""

    def __init__(self, pages, entries_per_block, record_bytes, stride, device, align=None):
        payload = entries_per_block * record_bytes
        self.entries_per_block = int(entries_per_block)
        if self.entries_per_block <= 0:
            raise ValueError("entries_per_block must be positive")
        self.stride = int(stride or (payload if align is None else _round_up(payload, align)))
        if self.stride < payload:
            raise ValueError("block stride does not cover its payload")
        self.data = torch.zeros(pages, self.stride, dtype=torch.uint8, device=device)
        self._free = list(range(pages - 1, -1, -1))

    def take(self):
        return self._free.pop()

    def give_back(self, pages):
        self._free.extend(reversed(pages))

    def entry(self, table, index):
        """Destination of logical entry `index` of a request; grows its page table."""
        page = index // self.entries_per_block
        while len(table) <= page:
            table.append(self.take())
        return table[page] * self.entries_per_block + index % self.entries_per_block


class KVCacheManager:
    def __init__(self, capacity, pages_per_pool, max_pages_per_req, device="cuda", state_ring_entries=MIN_RING,
                 idx_entries_per_block=TOKENS_PER_BLOCK // RATIO, cmp_entries_per_block=TOKENS_PER_BLOCK // RATIO,
                 swa_entries_per_block=TOKENS_PER_BLOCK, indexer_fp8=True, idx_block_stride_bytes=None,
                 cmp_block_stride_bytes=None, swa_block_stride_bytes=None):
        if state_ring_entries < MIN_RING:
            raise ValueError("state ring must cover the 8-entry overlap window")
        self.state_ring_entries = int(state_ring_entries)
        self.indexer_fp8 = bool(indexer_fp8)
        self.idx_entry_bytes = IDX_DIM + 4 if indexer_fp8 else IDX_DIM // 2 + 4
        self.capacity, self.max_pages, self.device = capacity, max_pages_per_req, device
        self._pools = {
            "swa": _PagePool(pages_per_pool, swa_entries_per_block, M1_RECORD, swa_block_stride_bytes, device, 576),
            "cmp": _PagePool(pages_per_pool, cmp_entries_per_block, M1_RECORD, cmp_block_stride_bytes, device, 576),
            "idx": _PagePool(pages_per_pool, idx_entries_per_block, self.idx_entry_bytes, idx_block_stride_bytes, device),
        }
        self.entries_per_block = {k: p.entries_per_block for k, p in self._pools.items()}
        self.block_stride_bytes = {k: p.stride for k, p in self._pools.items()}
        self.swa_pool, self.cmp_pool, self.idx_pool = (self._pools[k].data for k in ("swa", "cmp", "idx"))
        self.main_state = torch.empty(capacity, self.state_ring_entries, 2048, dtype=torch.float32, device=device)
        self.idx_state = torch.empty(capacity, self.state_ring_entries, 512, dtype=torch.float32, device=device)
        for slot in range(capacity):
            self._reset_state(slot)
        self._free_slots = list(range(capacity - 1, -1, -1))
        self.reqs = {}          # slot -> {"pos": last position, "swa"/"cmp"/"idx": page tables}

    # ---- slot lifecycle: a new or reused slot starts with kv = 0, score = -inf
    def _reset_state(self, slot):
        for state, half in ((self.main_state, 1024), (self.idx_state, 256)):
            state[slot, :, :half] = 0.0
            state[slot, :, half:] = NEG_INF

    def alloc_request(self):
        slot = self._free_slots.pop()
        self._reset_state(slot)
        swa = self._pools["swa"]
        window_pages = -(-WIN // swa.entries_per_block)
        self.reqs[slot] = {"pos": -1, "cmp": [], "idx": [], "swa": [swa.take() for _ in range(window_pages)]}
        return slot

    def advance(self, slot, tokens):
        """Bookkeeping of a prefill of `tokens` tokens (not in the reference's manager): moves the
        request's position forward and takes the pages its compressed entries occupy, without
        producing per-token destinations.  The caches themselves are filled by whoever prefills."""
        req = self.reqs[slot]
        req["pos"] += int(tokens)
        entries = (req["pos"] + 1) // RATIO
        if entries:
            for name in ("idx", "cmp"):
                self._pools[name].entry(req[name], entries - 1)

    def free_request(self, slot):
        req = self.reqs.pop(slot)
        for name in ("swa", "cmp", "idx"):
            self._pools[name].give_back(req[name])
        self._free_slots.append(slot)

    # ---- one decode step: positions, state rows and cache destinations of every request
    def step_begin(self, slots):
        pos, idx_dst, cmp_dst, swa_dst = [], [], [], []
        swa = self._pools["swa"]
        for s in slots:
            req = self.reqs[s]
            req["pos"] += 1
            p = req["pos"]
            pos.append(p)
            ring = p % WIN
            swa_dst.append(req["swa"][ring // swa.entries_per_block] * swa.entries_per_block + ring % swa.entries_per_block)
            if (p + 1) % RATIO == 0:                 # this token completes compressed entry ct
                ct = (p + 1) // RATIO - 1
                idx_dst.append(self._pools["idx"].entry(req["idx"], ct))
                cmp_dst.append(self._pools["cmp"].entry(req["cmp"], ct))
            else:
                idx_dst.append(-1)
                cmp_dst.append(-1)
        i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=self.device)
        rows = self.state_rows(slots, pos)
        return dict(slots=list(slots), pos=i64(pos), q_pos=torch.tensor(pos, dtype=torch.int32, device=self.device),
                    main_state_row=rows, idx_state_row=rows.clone(), idx_dst=i64(idx_dst), cmp_dst=i64(cmp_dst),
                    swa_dst=i64(swa_dst))

    def state_rows(self, slots, pos):
        """Row of the folded [capacity * ring, width] state view: slot * ring + pos % ring."""
        p = np.asarray([int(x) for x in pos], dtype=np.int64) % self.state_ring_entries
        s = np.asarray(list(slots), dtype=np.int64)
        return torch.from_numpy(s * self.state_ring_entries + p).to(self.device)

    main_state_rows = state_rows

    def block_table(self, name, slots):
        bt = np.zeros((len(slots), self.max_pages), np.int32)
        for i, s in enumerate(slots):
            tab = self.reqs[s][name]
            bt[i, :len(tab)] = tab
        return torch.from_numpy(bt).to(self.device)

    def geometry(self, name):
        return dict(entries_per_block=self.entries_per_block[name], block_stride_bytes=self.block_stride_bytes[name])

    def n_compressed(self, slots, pos):
        return torch.tensor([(int(p) + 1) // RATIO for p in pos], dtype=torch.int32, device=self.device)

    def swa_indices(self, slots, pos, swa_topk):
        """[B, 1, swa_topk] pool entries of the last min(swa_topk, pos + 1) tokens through the
        ring (token t sits at ring slot t % 128), -1 padded, and how many are valid."""
        out = np.full((len(slots), 1, swa_topk), -1, np.int32)
        lens = np.zeros(len(slots), np.int32)
        epb = self.entries_per_block["swa"]
        for i, s in enumerate(slots):
            p = int(pos[i])
            n = min(swa_topk, p + 1)
            ring = np.arange(p + 1 - n, p + 1) % WIN
            table = np.asarray(self.reqs[s]["swa"], np.int64)
            out[i, 0, :n] = table[ring // epb] * epb + ring % epb
            lens[i] = n
        return torch.from_numpy(out).to(self.device), torch.from_numpy(lens).to(self.device)

    # ---- views for the consumers
    def model1_cache_view(self, name):
        """[pages, entries, 1, 584] float8 view of a MODEL1 pool (sparse-attention layout)."""
        pool = self._pools[name]
        return pool.data.as_strided((pool.data.size(0), pool.entries_per_block, 1, M1_RECORD),
                                    (pool.stride, M1_RECORD, M1_RECORD, 1)).view(torch.float8_e4m3fn)

    def indexer_cache_view(self):
        """[pages, entries, 1, 132] logical view of the FP8 indexer pool; physically a page is all
        key bytes, then all fp32 scales (the layout wuda_mqa_logits_fp8 takes as kv_pages)."""
        if not self.indexer_fp8:
            raise ValueError("FP8 indexer cache view requested for an FP4 pool")
        pool = self._pools["idx"]
        return pool.data.as_strided((pool.data.size(0), pool.entries_per_block, 1, self.idx_entry_bytes),
                                    (pool.stride, self.idx_entry_bytes, self.idx_entry_bytes, 1))
