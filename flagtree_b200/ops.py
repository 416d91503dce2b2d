"""Python call surface of the hot path: same call shapes as the reference's kernel wrappers.

Every function here only validates arguments, allocates outputs with torch and forwards plain
pointers to the C ABI (include/flagtree_b200.h).  There is no PyTorch or CPU fallback: if the
shared library is missing the call raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

D_QK = 576
D_V = 512


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            # The reference's launcher raises ValueError for host tensors
            # (third_party/nvidia/backend/driver.py:259-264).
            raise ValueError("Pointer argument cannot be accessed from the device: expected CUDA tensors")


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _auto_splits(s_q: int, topk: int, device) -> int:
    """Split the top-k axis when there are too few query tokens to fill the SMs (decode)."""
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = max(1, (topk + 63) // 64)
    if 2 * s_q >= sms:
        return 1
    return int(max(1, min(16, sms // (2 * s_q), tiles)))


def _split_workspace(a, s_q: int, h: int, n_splits: int, device):
    """Fills the split fields of the argument struct; returns the scratch tensor (kept alive by the caller)."""
    a.n_splits = n_splits
    if n_splits <= 1:
        a.workspace, a.workspace_bytes = None, 0
        return None
    nbytes = int(_lib.load().ftb_sparse_mla_workspace_bytes(s_q, h, n_splits))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), nbytes
    return ws


def _check_status(status: Optional[torch.Tensor], what: str):
    if status is None:
        return
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: device status {_lib.STATUS_NAMES.get(code, code)}")


def sparse_mla_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                   sm_scale: Optional[float] = None, d_v: int = D_V, *, lse_base2: bool = False,
                   out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                   check: bool = False, algo: int = 0, num_splits: Optional[int] = None,
                   _dbg_scores: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Top-k sparse MLA forward.

    q [S_q, h, 576] bf16, kv [S_kv, 576] (or [S_kv, 1, 576]) bf16, indices [S_q, topk] int32 with
    -1 padding.  Returns (out [S_q, h, 512] bf16, lse [S_q, h] fp32, natural log).  Takes over
    the reference's decode_attention_fwd launch pair
    (third_party/mthreads/python/test/wmma/test_accuracy_musa_vllm_mla.py:571-620) with the
    token table as `indices`.  `sm_scale` defaults to 576**-0.5 (:640 of the same file).
    `check=True` reads back the device status word (one host sync) and raises on a bad index
    or a device-side timeout.  `num_splits` > 1 splits the top-k axis over several CTAs and merges the
    partial results (the reference's NUM_KV_SPLITS stage 2); it selects the single-CTA kernel.
    """
    _require_cuda(q, kv, indices)
    if kv.dim() == 3:
        assert kv.shape[1] == 1, "latent KV has a single shared head"
        kv = kv[:, 0, :]
    assert q.dim() == 3 and kv.dim() == 2 and indices.dim() == 2, "expected q[S_q,h,576], kv[S_kv,576], indices[S_q,topk]"
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16, "q and kv must be bf16"
    assert indices.dtype == torch.int32, "indices must be int32"
    assert q.shape[2] == D_QK and kv.shape[1] == D_QK, "q/k head dim must be 576 (512 latent + 64 rope)"
    assert d_v == D_V, "v head dim must be 512"
    assert indices.shape[0] == q.shape[0]
    assert q.stride(2) == 1 and kv.stride(1) == 1 and indices.stride(1) == 1, "innermost dimension must be contiguous"
    s_q, h, _ = q.shape
    if sm_scale is None:
        sm_scale = D_QK ** -0.5
    if out is None:
        out = torch.empty(s_q, h, D_V, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(s_q, h, dtype=torch.float32, device=q.device)
    assert out.shape == (s_q, h, D_V) and out.dtype == torch.bfloat16 and out.stride(2) == 1
    assert lse.shape == (s_q, h) and lse.dtype == torch.float32 and lse.stride(1) == 1
    status = torch.zeros(1, dtype=torch.int32, device=q.device) if check else None
    lib = _lib.load()
    for h0 in range(0, h, 128):      # more than 128 heads: one launch per block of 128 heads
        h1 = min(h, h0 + 128)
        qs, os_, ls = q[:, h0:h1], out[:, h0:h1], lse[:, h0:h1]
        a = _lib.SparseMlaArgs()
        a.q, a.kv, a.indices = qs.data_ptr(), kv.data_ptr(), indices.data_ptr()
        a.out, a.lse = os_.data_ptr(), ls.data_ptr()
        a.s_q, a.h, a.s_kv, a.topk = s_q, h1 - h0, kv.shape[0], indices.shape[1]
        a.q_stride_token, a.q_stride_head = qs.stride(0), qs.stride(1)
        a.kv_stride_row = kv.stride(0)
        a.idx_stride_token = indices.stride(0)
        a.out_stride_token, a.out_stride_head = os_.stride(0), os_.stride(1)
        a.lse_stride_token = ls.stride(0)
        a.sm_scale, a.lse_base2, a.algo_id = float(sm_scale), int(lse_base2), int(algo)
        a.status = status.data_ptr() if status is not None else None
        a.kv_is_fp8 = 0
        a.dbg_scores = _dbg_scores.data_ptr() if _dbg_scores is not None else None
        _ws = _split_workspace(a, s_q, h1 - h0, int(num_splits) if num_splits else 1, q.device)
        with torch.cuda.device(q.device):
            rc = lib.ftb_sparse_mla_fwd(C.byref(a), C.c_void_p(_stream_ptr(q.device)))
        _lib.check(rc, "sparse_mla_fwd")
    _check_status(status, "sparse_mla_fwd")
    return out, lse


_HOST_PIPES = {}


def sparse_mla_fwd_host(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: Optional[float] = None,
                        *, out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
                        device: Optional[torch.device] = None, chunk_tokens: int = 512
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """`sparse_mla_fwd` for HOST tensors (the form a plugin boundary with host buffers needs): q [S_q, h, 576]
    bf16, kv [S_kv, 576] bf16, indices [S_q, topk] int32 and the results out [S_q, h, 512] bf16, lse [S_q, h]
    fp32 live in host memory (pinned memory makes the copies asynchronous).  The query tokens go through the
    device in chunks of `chunk_tokens` on three streams: the host-to-device copy of chunk i + 1, the kernel of
    chunk i and the device-to-host copy of chunk i - 1 run at the same time, so that a step costs about the
    longer of the two copy directions instead of their sum plus the kernel.  The current stream waits for the
    last copy; the caller synchronises it before reading `out` (as after any asynchronous copy)."""
    assert not q.is_cuda and not kv.is_cuda and not indices.is_cuda, "host tensors expected"
    assert q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and indices.dtype == torch.int32
    if kv.dim() == 3:
        kv = kv.reshape(kv.shape[0], -1)
    s_q, h, _ = q.shape
    topk = indices.shape[1]
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    if sm_scale is None:
        sm_scale = D_QK ** -0.5
    if out is None:
        out = torch.empty(s_q, h, D_V, dtype=torch.bfloat16, pin_memory=True)
    if lse is None:
        lse = torch.empty(s_q, h, dtype=torch.float32, pin_memory=True)
    ct = max(1, min(int(chunk_tokens), s_q))
    key = (dev.index, ct, h, topk, kv.shape[0])
    pipe = _HOST_PIPES.get(key)
    if pipe is None:
        with torch.cuda.device(dev):
            pipe = {
                "q": [torch.empty(ct, h, D_QK, dtype=torch.bfloat16, device=dev) for _ in range(2)],
                "idx": [torch.empty(ct, topk, dtype=torch.int32, device=dev) for _ in range(2)],
                "out": [torch.empty(ct, h, D_V, dtype=torch.bfloat16, device=dev) for _ in range(2)],
                "lse": [torch.empty(ct, h, dtype=torch.float32, device=dev) for _ in range(2)],
                "kv": torch.empty(kv.shape[0], D_QK, dtype=torch.bfloat16, device=dev),
                "s_in": torch.cuda.Stream(dev), "s_c": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
            }
        _HOST_PIPES[key] = pipe
    s_in, s_c, s_out = pipe["s_in"], pipe["s_c"], pipe["s_out"]
    cur = torch.cuda.current_stream(dev)
    for s in (s_in, s_c, s_out):
        s.wait_stream(cur)          # nothing of this call overtakes earlier work of the caller's stream
    ev_in = [None, None]            # chunk landed in staging buffer b
    ev_c = [None, None]             # kernel on staging buffer b finished (its inputs may be overwritten)
    ev_out = [None, None]           # results of staging buffer b are on their way home (dout[b] may be overwritten)
    with torch.cuda.stream(s_in):
        pipe["kv"].copy_(kv, non_blocking=True)
    n_chunks = (s_q + ct - 1) // ct
    for i in range(n_chunks):
        b = i & 1
        lo, hi = i * ct, min(s_q, (i + 1) * ct)
        n = hi - lo
        with torch.cuda.stream(s_in):
            if ev_c[b] is not None:
                s_in.wait_event(ev_c[b])
            pipe["q"][b][:n].copy_(q[lo:hi], non_blocking=True)
            pipe["idx"][b][:n].copy_(indices[lo:hi], non_blocking=True)
            ev_in[b] = s_in.record_event()
        with torch.cuda.stream(s_c):
            s_c.wait_event(ev_in[b])
            if ev_out[b] is not None:
                s_c.wait_event(ev_out[b])
            sparse_mla_fwd(pipe["q"][b][:n], pipe["kv"], pipe["idx"][b][:n], sm_scale, out=pipe["out"][b][:n],
                           lse=pipe["lse"][b][:n])
            ev_c[b] = s_c.record_event()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_c[b])
            out[lo:hi].copy_(pipe["out"][b][:n], non_blocking=True)
            lse[lo:hi].copy_(pipe["lse"][b][:n], non_blocking=True)
            ev_out[b] = s_out.record_event()
    cur.wait_stream(s_out)
    cur.wait_stream(s_c)
    cur.wait_stream(s_in)
    return out, lse


def sparse_mla_fwd_paged(q: torch.Tensor, kv_cache: torch.Tensor, kv_scale: torch.Tensor,
                         block_table: torch.Tensor, context_lens: torch.Tensor, indices: torch.Tensor,
                         sm_scale: Optional[float] = None, d_v: int = D_V, page_size: int = 64, *,
                         lse_base2: bool = False, check: bool = False, num_splits: Optional[int] = None,
                         two_pass: Optional[bool] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse MLA decode over a paged FP8 (e4m3) latent cache with one fp32 scale per page.

    q [B, n_q, h, 576] bf16; kv_cache [num_pages, page_size, 576] e4m3 (uint8 or float8_e4m3fn);
    kv_scale [num_pages] fp32 (value = fp8 * scale); block_table [B, max_pages] int32;
    context_lens [B] int32; indices [B, n_q, topk] int32 LOGICAL positions (-1 = padding).
    Physical row = block_table[b, p // page] * page + p % page, the addressing rule of
    test_accuracy_musa_vllm_mla.py:278-283.  Returns (out [B,n_q,h,512] bf16, lse [B,n_q,h] fp32).

    `two_pass`: convert the selected rows to a compact bf16 table first and run the persistent bf16 kernel on
    it (needs 1156 bytes of scratch per selected row); None = do so when the top-k axis is not split and the
    scratch stays below 4 GiB, False = the one-pass kernel that converts while it gathers.
    """
    _require_cuda(q, kv_cache, kv_scale, block_table, context_lens, indices)
    assert q.dim() == 4 and indices.dim() == 3 and kv_cache.dim() == 3
    assert q.dtype == torch.bfloat16
    assert kv_cache.dtype in (torch.uint8, torch.float8_e4m3fn), "kv_cache must hold e4m3 bytes"
    assert kv_cache.shape[1] == page_size and kv_cache.shape[2] == D_QK and kv_cache.is_contiguous()
    assert kv_scale.dtype == torch.float32 and kv_scale.numel() == kv_cache.shape[0] and kv_scale.is_contiguous()
    assert block_table.dtype == torch.int32 and context_lens.dtype == torch.int32 and indices.dtype == torch.int32
    assert block_table.stride(1) == 1 and context_lens.is_contiguous()
    assert d_v == D_V and q.shape[3] == D_QK
    b, n_q, h, _ = q.shape
    assert h <= 128, "at most 128 heads per call in the paged form"
    assert indices.shape[:2] == (b, n_q) and block_table.shape[0] == b and context_lens.shape[0] == b
    q2 = q.reshape(b * n_q, h, D_QK)
    idx2 = indices.reshape(b * n_q, indices.shape[2])
    assert q2.stride(2) == 1 and idx2.stride(1) == 1
    if sm_scale is None:
        sm_scale = D_QK ** -0.5
    out = torch.empty(b * n_q, h, D_V, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b * n_q, h, dtype=torch.float32, device=q.device)
    status = torch.zeros(1, dtype=torch.int32, device=q.device) if check else None
    a = _lib.SparseMlaArgs()
    a.q, a.kv, a.indices, a.out, a.lse = q2.data_ptr(), kv_cache.data_ptr(), idx2.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.s_q, a.h, a.s_kv, a.topk = b * n_q, h, kv_cache.shape[0] * page_size, idx2.shape[1]
    a.q_stride_token, a.q_stride_head = q2.stride(0), q2.stride(1)
    a.kv_stride_row = D_QK
    a.idx_stride_token = idx2.stride(0)
    a.out_stride_token, a.out_stride_head = out.stride(0), out.stride(1)
    a.lse_stride_token = lse.stride(0)
    a.sm_scale, a.lse_base2, a.algo_id = float(sm_scale), int(lse_base2), 0
    a.status = status.data_ptr() if status is not None else None
    a.kv_is_fp8 = 1
    a.kv_scale, a.block_table, a.context_lens = kv_scale.data_ptr(), block_table.data_ptr(), context_lens.data_ptr()
    a.page_size, a.q_per_seq, a.block_table_stride = page_size, n_q, block_table.stride(0)
    a.dbg_scores = None
    if num_splits is None:
        num_splits = _auto_splits(b * n_q, idx2.shape[1], q.device)
    _ws = _split_workspace(a, b * n_q, h, int(num_splits), q.device)
    if int(num_splits) <= 1 and two_pass is not False:
        need = int(_lib.load().ftb_sparse_mla_dequant_workspace_bytes(b * n_q, idx2.shape[1]))
        if two_pass or need <= (4 << 30):
            _ws = torch.empty(need, dtype=torch.uint8, device=q.device)
            a.workspace, a.workspace_bytes = _ws.data_ptr(), need
            a.algo_id = 6
    with torch.cuda.device(q.device):
        rc = _lib.load().ftb_sparse_mla_fwd(C.byref(a), C.c_void_p(_stream_ptr(q.device)))
    _lib.check(rc, "sparse_mla_fwd_paged")
    _check_status(status, "sparse_mla_fwd_paged")
    return out.view(b, n_q, h, D_V), lse.view(b, n_q, h)


def decode_attention_fwd(q, k_buffer, v_buffer, o, req_to_token, b_seq_len, attn_logits=None,
                         num_kv_splits=None, sm_scale=None, page_size=1, logit_cap=0.0, en_wmma=False):
    """Drop-in for the reference's `decode_attention_fwd` (test_accuracy_musa_vllm_mla.py:571-584)
    for the MLA shape (one shared latent head, Lk = 576, Lv = 512, page_size = 1): writes into `o`.

    `req_to_token [B, max_len]` is the token table and `b_seq_len [B]` the number of leading
    valid entries.  `attn_logits` and `num_kv_splits` are accepted and ignored (kv splitting is
    internal); when both are given the reference's shape assertion (:585) is kept.
    """
    if attn_logits is not None and num_kv_splits is not None:
        assert num_kv_splits == attn_logits.shape[2]
    assert page_size == 1, "the dense form takes a token table (page size 1); use sparse_mla_fwd_paged for pages"
    assert logit_cap == 0.0, "logit soft-capping is not part of the sparse MLA path"
    assert k_buffer.shape[-2] == 1 and k_buffer.shape[-1] == D_QK, "MLA form: one latent head of 576 dims"
    kv = k_buffer.reshape(-1, D_QK)
    assert v_buffer.shape[-1] == D_V
    topk = req_to_token.shape[1]
    pos = torch.arange(topk, device=req_to_token.device, dtype=torch.int32)
    idx = torch.where(pos[None, :] < b_seq_len[:, None].to(torch.int32), req_to_token.to(torch.int32),
                      torch.full((1, 1), -1, dtype=torch.int32, device=req_to_token.device))
    if sm_scale is None:
        sm_scale = D_QK ** -0.5
    sparse_mla_fwd(q, kv, idx.contiguous(), sm_scale, out=o)
    return o


def sparse_mla_merge(part_out: torch.Tensor, part_lse: torch.Tensor, *, lse_base2: bool = False,
                     out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Merge partial sparse-MLA results over disjoint sets of key/value rows by their log-sum-exps: the
    reference's second launch (`_decode_softmax_reducev_fwd`, test_accuracy_musa_vllm_mla.py:480-510, kernel
    :426-477) as an operation of its own.

    part_out [n_parts, S_q, h, 512] bf16 (outputs of `sparse_mla_fwd`) or fp32; part_lse [n_parts, S_q, h] fp32
    (natural log unless `lse_base2`; -inf marks a part without a valid row).  Returns (out [S_q, h, 512] bf16,
    lse [S_q, h] fp32).  Use: a context whose latent rows are sharded over GPUs -- every rank runs
    `sparse_mla_fwd` with `shard_indices(indices, lo, hi)`, the parts are all-gathered, this merges them."""
    _require_cuda(part_out, part_lse)
    assert part_out.dim() == 4 and part_lse.dim() == 3 and part_out.shape[3] == D_V
    assert part_out.dtype in (torch.bfloat16, torch.float32) and part_lse.dtype == torch.float32
    n_parts, s_q, h, _ = part_out.shape
    assert part_lse.shape == (n_parts, s_q, h)
    assert part_out.stride(3) == 1 and part_lse.stride(2) == 1, "innermost dimension must be contiguous"
    if out is None:
        out = torch.empty(s_q, h, D_V, dtype=torch.bfloat16, device=part_out.device)
    if lse is None:
        lse = torch.empty(s_q, h, dtype=torch.float32, device=part_out.device)
    assert out.shape == (s_q, h, D_V) and out.dtype == torch.bfloat16 and out.stride(2) == 1
    assert lse.shape == (s_q, h) and lse.dtype == torch.float32 and lse.stride(1) == 1
    a = _lib.SparseMlaMergeArgs()
    a.part_out, a.part_lse, a.out, a.lse = part_out.data_ptr(), part_lse.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.s_q, a.h, a.n_parts = s_q, h, n_parts
    a.part_is_fp32, a.lse_base2 = int(part_out.dtype == torch.float32), int(lse_base2)
    a.part_stride_part, a.part_stride_token, a.part_stride_head = part_out.stride(0), part_out.stride(1), part_out.stride(2)
    a.lse_stride_part, a.lse_stride_part_token = part_lse.stride(0), part_lse.stride(1)
    a.out_stride_token, a.out_stride_head, a.lse_stride_token = out.stride(0), out.stride(1), lse.stride(0)
    with torch.cuda.device(part_out.device):
        rc = _lib.load().ftb_sparse_mla_merge(C.byref(a), C.c_void_p(_stream_ptr(part_out.device)))
    _lib.check(rc, "sparse_mla_merge")
    return out, lse


def shard_indices(indices: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Index list of a rank that holds latent rows [lo, hi) of the context: entries inside the range become
    local row numbers, all others -1 (padding).  The -1 entries may sit anywhere in the list."""
    inside = (indices >= lo) & (indices < hi)
    return torch.where(inside, indices - lo, torch.full_like(indices, -1))


def topk_indices(scores: torch.Tensor, topk: int, lengths: Optional[torch.Tensor] = None, *,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The index producer in front of `sparse_mla_fwd`: scores [S_q, S_kv] fp32 -> indices [S_q, topk] int32, per
    token the positions of the `topk` largest scores among its first `lengths[t]` positions (all of them when
    `lengths` is None), ascending, padded with -1.  Exact: floats ordered by value with -0 below +0 and NaN above
    +inf, ties to the lower position.  The reference builds index lists for its block-sparse ops on the device
    in the same spirit (python/triton/ops/blocksparse/matmul.py:117-127)."""
    _require_cuda(scores, lengths)
    assert scores.dim() == 2 and scores.dtype == torch.float32 and scores.stride(1) == 1
    s_q, s_kv = scores.shape
    if lengths is not None:
        assert lengths.dtype == torch.int32 and lengths.shape == (s_q,) and lengths.is_contiguous()
    if out is None:
        out = torch.empty(s_q, topk, dtype=torch.int32, device=scores.device)
    assert out.shape == (s_q, topk) and out.dtype == torch.int32 and out.stride(1) == 1
    a = _lib.TopkArgs()
    a.scores, a.out = scores.data_ptr(), out.data_ptr()
    a.lengths = lengths.data_ptr() if lengths is not None else None
    a.s_q, a.s_kv, a.topk = s_q, s_kv, int(topk)
    a.scores_stride_token, a.out_stride_token = scores.stride(0), out.stride(0)
    with torch.cuda.device(scores.device):
        rc = _lib.load().ftb_topk_indices(C.byref(a), C.c_void_p(_stream_ptr(scores.device)))
    _lib.check(rc, "topk_indices")
    return out


def kv_cache_write_fp8(rows: torch.Tensor, slot_mapping: torch.Tensor, kv_cache: torch.Tensor, kv_scale: torch.Tensor,
                       page_size: int = 64, *, check: bool = False) -> None:
    """Quantise new latent rows to e4m3 with one fp32 scale per page and scatter them into the paged cache, in
    place: the producer of the format `sparse_mla_fwd_paged` reads.  Analogue of the reference's quantising
    cache writer `destindex_copy_quantize_int4kv_init`
    (third_party/hcu/python/test/unit/sglang/decode_attention_int4kv.py:934).

    rows [n, 576] bf16; slot_mapping [n] int32, slot = page * page_size + position (-1 skips the row; slots of
    one call must be distinct); kv_cache [num_pages, page_size, 576] e4m3 bytes; kv_scale [num_pages] fp32, 0 for
    a page that holds nothing yet.  A page's scale only grows: max(old, max|new rows| / 448); when it grows for
    a page that already held rows, those bytes are requantised to the new scale first."""
    _require_cuda(rows, slot_mapping, kv_cache, kv_scale)
    assert rows.dim() == 2 and rows.shape[1] == D_QK and rows.dtype == torch.bfloat16 and rows.stride(1) == 1
    assert slot_mapping.dtype == torch.int32 and slot_mapping.shape == (rows.shape[0],) and slot_mapping.is_contiguous()
    assert kv_cache.dtype in (torch.uint8, torch.float8_e4m3fn) and kv_cache.is_contiguous()
    assert kv_cache.dim() == 3 and kv_cache.shape[1] == page_size and kv_cache.shape[2] == D_QK
    assert kv_scale.dtype == torch.float32 and kv_scale.shape == (kv_cache.shape[0],) and kv_scale.is_contiguous()
    lib = _lib.load()
    num_pages = kv_cache.shape[0]
    ws = torch.empty(int(lib.ftb_kv_cache_write_workspace_bytes(num_pages)), dtype=torch.uint8, device=rows.device)
    status = torch.zeros(1, dtype=torch.int32, device=rows.device) if check else None
    a = _lib.KvCacheWriteArgs()
    a.rows, a.slot_mapping, a.kv_cache, a.kv_scale = rows.data_ptr(), slot_mapping.data_ptr(), kv_cache.data_ptr(), kv_scale.data_ptr()
    a.n_rows, a.num_pages, a.page_size = rows.shape[0], num_pages, page_size
    a.row_stride = rows.stride(0)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.status = status.data_ptr() if status is not None else None
    with torch.cuda.device(rows.device):
        rc = lib.ftb_kv_cache_write_fp8(C.byref(a), C.c_void_p(_stream_ptr(rows.device)))
    _lib.check(rc, "kv_cache_write_fp8")
    _check_status(status, "kv_cache_write_fp8")


# ------------------------------------------------------------------------------------- GEMM
def matmul(a: torch.Tensor, b: torch.Tensor, acc_dtype=None, input_precision=None, fp8_fast_accum=True,
           output_dtype=None, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A @ B for bf16 operands with fp32 accumulation; same call shape as the reference's
    `triton.ops.matmul` (python/triton/ops/matmul.py:231-236).  Non-contiguous inputs are copied as
    the reference does (:165-168); the shape check is the reference's assertion (:170)."""
    _require_cuda(a, b)
    if a.stride(0) > 1 and a.stride(1) > 1:
        a = a.contiguous()
    if b.stride(0) > 1 and b.stride(1) > 1:
        b = b.contiguous()
    assert a.shape[1] == b.shape[0], "incompatible dimensions"
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands only"
    assert acc_dtype in (None, torch.float32), "bf16 inputs accumulate in fp32"
    assert output_dtype in (None, torch.bfloat16)
    if a.stride(1) != 1:
        a = a.contiguous()
    if b.stride(1) != 1:
        b = b.contiguous()
    m, k = a.shape
    n = b.shape[1]
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    _gemm_into(a, b, out)
    return out


def _gemm_into(a, b, c, status=None):
    g = _lib.GemmArgs()
    g.a, g.b, g.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    g.m, g.n, g.k = a.shape[0], b.shape[1], a.shape[1]
    g.lda, g.ldb, g.ldc = a.stride(0), b.stride(0), c.stride(0)
    g.status = status.data_ptr() if status is not None else None
    with torch.cuda.device(a.device):
        rc = _lib.load().ftb_gemm_bf16(C.byref(g), C.c_void_p(_stream_ptr(a.device)))
    _lib.check(rc, "matmul")


def matmul_fp8_blockscaled(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor, *,
                           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = (A * a_scale) @ (B * b_scale) for e4m3 operands (uint8 or float8_e4m3fn storage) with 1x128 (A) and
    128x128 (B) fp32 block scales; bf16 result.  Operands follow the reference's fp8 matmul convention of
    raw 8-bit patterns (python/test/unit/operators/test_matmul.py:165-169)."""
    _require_cuda(a, a_scale, b, b_scale)
    for t in (a, b):
        assert t.dtype in (torch.uint8, torch.float8_e4m3fn), "operands must hold e4m3 bytes"
    assert a.shape[1] == b.shape[0], "incompatible dimensions"
    m, k = a.shape
    n = b.shape[1]
    assert k % 128 == 0 and n % 128 == 0, "k and n must be multiples of the 128-wide scale blocks"
    assert a_scale.shape == (m, k // 128) and b_scale.shape == (k // 128, n // 128)
    assert a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32
    assert a.stride(1) == 1 and a_scale.stride(1) == 1 and b_scale.stride(1) == 1
    # b may be a [K, N] row-major matrix or the transposed view `w.t()` of a weight kept as [N, K] (K contiguous),
    # which the tensor cores read as the K-major operand
    b_kmajor = b.stride(1) != 1
    assert b.stride(1) == 1 or b.stride(0) == 1, "b must be contiguous along N or along K"
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    g = _lib.GemmFp8Args()
    g.a, g.b, g.c, g.a_scale, g.b_scale = a.data_ptr(), b.data_ptr(), out.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr()
    g.m, g.n, g.k = m, n, k
    g.lda, g.ldb, g.ldc = a.stride(0), (b.stride(1) if b_kmajor else b.stride(0)), out.stride(0)
    g.a_scale_ld, g.b_scale_ld = a_scale.stride(0), b_scale.stride(0)
    g.status = None
    g.b_kmajor = 1 if b_kmajor else 0
    with torch.cuda.device(a.device):
        rc = _lib.load().ftb_gemm_fp8_blockscaled(C.byref(g), C.c_void_p(_stream_ptr(a.device)))
    _lib.check(rc, "matmul_fp8_blockscaled")
    return out


class GemmRsContext:
    """Workspace of one (M, N, group) GEMM + reduce-scatter shape: peer-mapped receive slots and flags.

    Creation is collective over `group`.  One call may be in flight per context.  `fp8=True` announces that the
    context will serve block-scaled FP8 calls (`fp8()`), which keeps "auto" off the copy-engine protocol: its flag
    words differ from those of the FP8 form.
    """

    def __init__(self, m: int, n: int, group=None, device: Optional[torch.device] = None, provider: str = "auto",
                 protocol: str = "auto", fp8: bool = False):
        import torch.distributed as dist
        from .symm import SymmetricBuffer
        self.group = group
        self.rank = dist.get_rank(group)
        self.tp = dist.get_world_size(group)
        self.m, self.n = m, n
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        lib = _lib.load()
        rb, fb = C.c_int64(), C.c_int64()
        _lib.check(lib.ftb_gemm_rs_workspace_bytes(m, n, self.tp, C.byref(rb), C.byref(fb)), "gemm_rs workspace")
        with torch.cuda.device(self.device):
            self.recv = SymmetricBuffer(rb.value, group, self.device, provider)
            self.flags = SymmetricBuffer(fb.value, group, self.device, provider)
            recv_ptrs = (C.c_void_p * self.tp)(*self.recv.ptrs)
            flag_ptrs = (C.c_void_p * self.tp)(*self.flags.ptrs)
            ctx = C.c_void_p()
            _lib.check(lib.ftb_gemm_rs_ctx_create(C.byref(ctx), self.rank, self.tp, m, n, recv_ptrs, flag_ptrs),
                       "gemm_rs ctx_create")
        self._ctx = ctx
        # Pull protocol (in-switch reduction) when every rank obtained a multicast mapping, else push.
        import torch.distributed as dist
        # measured at the cfg4 per-rank shape: push 0.311 ms against pull 0.36-0.39 at tp = 2, level at tp = 4,
        # pull 0.383-0.390 against push 0.463-0.471 at tp = 8; so "auto" pulls from four ranks on
        # "auto" for bf16 calls: the copy-engine exchange at two ranks (0.230 ms against pull 0.317, push 0.30 and
        # GEMM + NCCL 0.358), the in-switch reduction from four ranks on (0.320 ms against copy 0.341 and NCCL 0.379
        # at tp = 4: the copy engines of a rank move about 500 GB/s, too little for three or seven shards)
        if protocol == "auto" and not fp8 and self.tp <= 2:
            protocol = "copy"
        want_pull = protocol == "pull" or (protocol == "auto" and self.tp >= 4)
        have_mc = torch.tensor([1 if (self.recv.mc_ptr and want_pull) else 0], device=self.device)
        dist.all_reduce(have_mc, op=dist.ReduceOp.MIN, group=group)
        self.protocol = "pull" if int(have_mc.item()) == 1 else "push"
        if protocol == "pull" and self.protocol != "pull":
            raise RuntimeError("gemm_rs: protocol='pull' needs an NVSwitch multicast mapping on every rank")
        # "staged" = GEMM per group of shards + one reduce kernel at the end (in-switch reduction when there is a
        # multicast mapping, peer loads otherwise); "push" / "pull" = the fused kernel.  Measured at the cfg4
        # per-rank shape the staged form is the slowest (0.44 ms at tp = 2, 0.48 ms at tp = 8), so "auto"
        # keeps the fused kernel; the FP8 form always runs staged.
        self.staged = protocol == "staged"
        # "copy" = one GEMM launch; the other ranks' row shards leave in pieces by device-to-device copies on a second
        # stream as they complete (copy engines), the epilogue of the own rows adds the peers' partials
        if protocol == "copy":
            _lib.check(lib.ftb_gemm_rs_ctx_set_copy_engine(ctx, 1), "gemm_rs set_copy_engine")
            self.protocol = "copy"
        have_mc_any = torch.tensor([1 if self.recv.mc_ptr else 0], device=self.device)
        dist.all_reduce(have_mc_any, op=dist.ReduceOp.MIN, group=group)
        if protocol != "copy" and (self.protocol == "pull" or (self.staged and int(have_mc_any.item()) == 1)):
            _lib.check(lib.ftb_gemm_rs_ctx_set_multicast(ctx, C.c_void_p(self.recv.mc_ptr)), "gemm_rs set_multicast")
        if self.staged:
            _lib.check(lib.ftb_gemm_rs_ctx_set_staged(ctx, 1), "gemm_rs set_staged")
            self.protocol = "staged"
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def __call__(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(a, b)
        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        assert a.shape[0] == self.m and b.shape[1] == self.n and a.shape[1] == b.shape[0], "incompatible dimensions"
        assert a.stride(1) == 1 and b.stride(1) == 1
        if out is None:
            out = torch.empty(self.m // self.tp, self.n, dtype=torch.bfloat16, device=a.device)
        assert out.shape == (self.m // self.tp, self.n) and out.stride(1) == 1
        with torch.cuda.device(a.device):
            rc = _lib.load().ftb_gemm_rs(self._ctx, a.data_ptr(), b.data_ptr(), out.data_ptr(), a.shape[1],
                                         a.stride(0), b.stride(0), out.stride(0), self.status.data_ptr(),
                                         C.c_void_p(_stream_ptr(a.device)))
        _lib.check(rc, "gemm_rs")
        return out

    def fp8(self, a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Block-scaled FP8 form: A_r [M, K/tp] e4m3 with fp32 scales [M, (K/tp)/128], B_r [K/tp, N] e4m3 with
        fp32 scales [(K/tp)/128, N/128]; returns this rank's rows of the sum of the dequantised products as
        bf16.  A context serves either bf16 calls or FP8 calls."""
        _require_cuda(a, a_scale, b, b_scale)
        if self.protocol == "copy":
            raise RuntimeError("gemm_rs_fp8: this context runs the copy-engine protocol of the bf16 form; create it with fp8=True")
        for t in (a, b):
            assert t.dtype in (torch.uint8, torch.float8_e4m3fn), "operands must hold e4m3 bytes"
        assert a.shape[0] == self.m and b.shape[1] == self.n and a.shape[1] == b.shape[0], "incompatible dimensions"
        k = a.shape[1]
        assert k % 128 == 0 and self.n % 128 == 0, "k and n must be multiples of the 128-wide scale blocks"
        assert a_scale.shape == (self.m, k // 128) and b_scale.shape == (k // 128, self.n // 128)
        assert a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32
        assert a.stride(1) == 1 and b.stride(1) == 1 and a_scale.stride(1) == 1 and b_scale.stride(1) == 1
        if out is None:
            out = torch.empty(self.m // self.tp, self.n, dtype=torch.bfloat16, device=a.device)
        assert out.shape == (self.m // self.tp, self.n) and out.stride(1) == 1
        with torch.cuda.device(a.device):
            rc = _lib.load().ftb_gemm_rs_fp8(self._ctx, a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(),
                                             out.data_ptr(), k, a.stride(0), b.stride(0), a_scale.stride(0),
                                             b_scale.stride(0), out.stride(0), self.status.data_ptr(),
                                             C.c_void_p(_stream_ptr(a.device)))
        _lib.check(rc, "gemm_rs_fp8")
        return out

    def set_wait_limit(self, cycles: int):
        """Longest device-side wait for another rank, in SM clock cycles (default about one second)."""
        _lib.check(_lib.load().ftb_gemm_rs_ctx_set_wait_limit(self._ctx, int(cycles)), "gemm_rs set_wait_limit")

    def check(self):
        """Reads the device status word (one host synchronisation) and raises RuntimeError on a timeout.  After a
        timeout the context is dead on every rank: close it and create a new one."""
        _check_status(self.status, "gemm_rs")

    def close(self):
        """Collective over the group.  A peer's kernel may still read this rank's partial or store its `done`
        word into this rank's flags after this rank's own stream has drained, so the buffers are only released
        between two barriers: every rank idle, peers' mappings closed, then the memory itself."""
        if self._ctx is not None:
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            _lib.load().ftb_gemm_rs_ctx_destroy(self._ctx)
            self._ctx = None
            self.recv.close_peers()
            self.flags.close_peers()
            dist.barrier(self.group)
            self.recv.close()
            self.flags.close()


class AgGemmContext:
    """Workspace of one (M, K, group) all-gather + GEMM shape: peer-mapped gather buffers [M, K] and flags.
    Creation and `close` are collective over `group`.  One call may be in flight per context."""

    def __init__(self, m: int, k: int, group=None, device: Optional[torch.device] = None, provider: str = "auto"):
        import torch.distributed as dist
        from .symm import SymmetricBuffer
        self.group = group
        self.rank = dist.get_rank(group)
        self.tp = dist.get_world_size(group)
        self.m, self.k = m, k
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        lib = _lib.load()
        ab, fb = C.c_int64(), C.c_int64()
        _lib.check(lib.ftb_ag_gemm_workspace_bytes(m, k, self.tp, C.byref(ab), C.byref(fb)), "ag_gemm workspace")
        with torch.cuda.device(self.device):
            self.ag = SymmetricBuffer(ab.value, group, self.device, provider)
            self.flags = SymmetricBuffer(fb.value, group, self.device, provider)
            ag_ptrs = (C.c_void_p * self.tp)(*self.ag.ptrs)
            flag_ptrs = (C.c_void_p * self.tp)(*self.flags.ptrs)
            ctx = C.c_void_p()
            _lib.check(lib.ftb_ag_gemm_ctx_create(C.byref(ctx), self.rank, self.tp, m, k, ag_ptrs, flag_ptrs), "ag_gemm ctx_create")
        self._ctx = ctx
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def __call__(self, a_shard: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(a_shard, b)
        assert a_shard.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
        assert a_shard.shape == (self.m // self.tp, self.k) and b.shape[0] == self.k, "incompatible dimensions"
        assert a_shard.stride(1) == 1 and b.stride(1) == 1
        n_local = b.shape[1]
        if out is None:
            out = torch.empty(self.m, n_local, dtype=torch.bfloat16, device=a_shard.device)
        assert out.shape == (self.m, n_local) and out.stride(1) == 1
        with torch.cuda.device(a_shard.device):
            rc = _lib.load().ftb_ag_gemm(self._ctx, a_shard.data_ptr(), b.data_ptr(), out.data_ptr(), n_local, a_shard.stride(0),
                                         b.stride(0), out.stride(0), self.status.data_ptr(), C.c_void_p(_stream_ptr(a_shard.device)))
        _lib.check(rc, "ag_gemm")
        return out

    def set_wait_limit(self, cycles: int):
        _lib.check(_lib.load().ftb_ag_gemm_ctx_set_wait_limit(self._ctx, int(cycles)), "ag_gemm set_wait_limit")

    def check(self):
        _check_status(self.status, "ag_gemm")

    def close(self):
        if self._ctx is not None:
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            _lib.load().ftb_ag_gemm_ctx_destroy(self._ctx)
            self._ctx = None
            self.ag.close_peers()
            self.flags.close_peers()
            dist.barrier(self.group)
            self.ag.close()
            self.flags.close()


_AG_CONTEXTS = {}


def ag_gemm(a_shard: torch.Tensor, b: torch.Tensor, group=None, *, out: Optional[torch.Tensor] = None,
            check: bool = False) -> torch.Tensor:
    """All-gather + GEMM: rank r passes its row shard A_r [M/tp, K] and its weight columns B_r [K, N_local] and gets
    C_r [M, N_local] = cat_r(A_r) @ B_r as bf16 (the column-parallel step that precedes `gemm_rs`).  Collective over
    `group`; the workspace of each (M, K, group) is created on first use and cached."""
    import torch.distributed as dist
    tp = dist.get_world_size(group)
    m, k = a_shard.shape[0] * tp, a_shard.shape[1]
    key = (m, k, a_shard.device.index, id(group))
    hit = _AG_CONTEXTS.get(key)
    if hit is None or hit[0] is not group:
        hit = _AG_CONTEXTS[key] = (group, AgGemmContext(m, k, group, a_shard.device))
    res = hit[1](a_shard, b, out)
    if check:
        hit[1].check()
    return res


_RS_CONTEXTS = {}     # (form, M, N, device, group key) -> (group, context); holding the group keeps its id unique


def _rs_context(form: str, m: int, n: int, group, device) -> "GemmRsContext":
    key = (form, m, n, device.index, id(group))
    hit = _RS_CONTEXTS.get(key)
    if hit is None or hit[0] is not group:
        hit = _RS_CONTEXTS[key] = (group, GemmRsContext(m, n, group, device, fp8=(form == "fp8")))
    return hit[1]


def gemm_rs_close_all():
    """Closes every workspace that `gemm_rs` / `gemm_rs_fp8` / `ag_gemm` created (collective over their groups)."""
    for key in sorted(_RS_CONTEXTS, key=lambda k: (k[0], k[1], k[2], k[3])):
        _RS_CONTEXTS[key][1].close()
    _RS_CONTEXTS.clear()
    for key in sorted(_AG_CONTEXTS, key=lambda k: (k[0], k[1], k[2])):
        _AG_CONTEXTS[key][1].close()
    _AG_CONTEXTS.clear()


def gemm_rs(a: torch.Tensor, b: torch.Tensor, group=None, *, out: Optional[torch.Tensor] = None,
            check: bool = False) -> torch.Tensor:
    """Row-parallel GEMM fused with reduce-scatter: rank r passes A_r [M, K/tp] and B_r [K/tp, N] and gets
    rows [r*M/tp, (r+1)*M/tp) of sum_r A_r @ B_r as bf16.  Collective over `group`; the workspace of each
    (M, N, group) is created on first use and cached (`gemm_rs_close_all` releases them).  `check=True` reads the
    device status word after the call (one host synchronisation) and raises on a device-side timeout."""
    ctx = _rs_context("bf16", a.shape[0], b.shape[1], group, a.device)
    res = ctx(a, b, out)
    if check:
        ctx.check()
    return res


def gemm_rs_fp8(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor, group=None, *,
                out: Optional[torch.Tensor] = None, check: bool = False) -> torch.Tensor:
    """Block-scaled FP8 form of `gemm_rs`: rank r passes A_r [M, K/tp] e4m3 with fp32 scales per 1 x 128 block
    ([M, (K/tp)/128]) and B_r [K/tp, N] e4m3 with fp32 scales per 128 x 128 block, and gets its rows of the sum of
    the dequantised products as bf16.  Workspaces are cached per (M, N, group), apart from those of `gemm_rs`."""
    ctx = _rs_context("fp8", a.shape[0], b.shape[1], group, a.device)
    res = ctx.fp8(a, a_scale, b, b_scale, out)
    if check:
        ctx.check()
    return res
