"""Mixed prefill + decode steps (jetfire_vllm/adapter/decode_path.py:1184-1284 gate,
:1402-1558 general split, :1561-1663 ordered split).

vLLM's scheduler may put sequences that decode one token and sequences that are being prefilled
into the same step.  The decode rows of such a step are served here from the packed cache
(``try_jetfire_decode`` on sub-selected metadata); the prefill rows, which attend only to the
keys and values of this very step, go to a variable-length attention over ``key`` / ``value``.

Two ways to find the rows:

* **ordered** -- the metadata carries the scheduler's own counts (``num_decodes``,
  ``num_prefills``, ``num_decode_tokens``, ``num_prefill_tokens``; decode sequences first) and
  says that no prefill row has cached context: plain slices, nothing read from the device;
* **general** -- ``query_start_loc`` and ``seq_lens`` are read back and every sequence with one
  query token is a decode row, wherever it stands.

Neither runs during stream capture: the decode part waits on the host for the correction.

Unlike the reference, which runs without vLLM's own KV cache and therefore has to raise when a
prefill row has cached context, this adapter leaves vLLM's cache in place: such a step is handed
back (None) and the caller's native attention serves it whole.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Callable, Sequence

import torch

from .config import JetFireConfig, get_jetfire_config
from .decode_path import try_jetfire_decode


@dataclass
class MixedSplit:
    """Which sequences of a step decode and which are prefilled, with their query rows."""
    decode_seqs: list[int] = field(default_factory=list)
    prefill_seqs: list[int] = field(default_factory=list)
    decode_rows: list[int] = field(default_factory=list)     # one query row per decode sequence
    prefill_rows: list[int] = field(default_factory=list)    # every query row of the prefill sequences
    prefill_cu: list[int] = field(default_factory=lambda: [0])   # cumulative lengths of the prefill sequences
    max_prefill_len: int = 0
    prefill_with_context: list[int] = field(default_factory=list)   # prefill sequences with seq_len > query_len
    ordered: bool = True     # decode sequences form a prefix of the step, prefill sequences the tail

    @property
    def mixed(self) -> bool:
        return bool(self.decode_seqs) and bool(self.prefill_seqs)


def split_mixed_batch(query_start_loc: Sequence[int], seq_lens: Sequence[int]) -> MixedSplit:
    """Classify the sequences of one step from host copies of ``query_start_loc`` (n + 1 entries)
    and ``seq_lens`` (n entries).  One query token = decode (also a sequence that vLLM counts as
    prefill because it has cached context but a single new token: attending its one token to the
    whole cached sequence is exactly a decode step, decode_path.py:1336-1399); more = prefill;
    none (padding) = skipped."""
    n = len(query_start_loc) - 1
    if n < 0 or len(seq_lens) < n:
        raise ValueError(f"query_start_loc has {n + 1} entries for {len(seq_lens)} sequence lengths")
    sp = MixedSplit()
    seen_prefill = False
    next_row = 0
    for i in range(n):
        lo, hi = int(query_start_loc[i]), int(query_start_loc[i + 1])
        qlen = hi - lo
        if qlen < 0:
            raise ValueError(f"query_start_loc decreases at sequence {i}")
        if qlen == 0:
            continue
        if lo != next_row:
            sp.ordered = False
        next_row = hi
        if qlen == 1:
            sp.decode_seqs.append(i)
            sp.decode_rows.append(lo)
            if seen_prefill:
                sp.ordered = False
        else:
            seen_prefill = True
            sp.prefill_seqs.append(i)
            sp.prefill_rows.extend(range(lo, hi))
            sp.prefill_cu.append(sp.prefill_cu[-1] + qlen)
            sp.max_prefill_len = max(sp.max_prefill_len, qlen)
            if int(seq_lens[i]) != qlen:
                sp.prefill_with_context.append(i)
    if sp.decode_seqs and sp.decode_seqs != list(range(sp.decode_seqs[0], sp.decode_seqs[0] + len(sp.decode_seqs))):
        sp.ordered = False
    return sp


def annotate_split_counts(metadata, query_start_loc_cpu, seq_lens_cpu):
    """Write the scheduler's split onto attention metadata when it is built (host tensors only,
    once per step rather than once per layer; JetFireAttentionMetadataBuilder.build of
    jetfire_vllm/adapter/jetfire_backend.py:66-127).  The counts are set only for a step whose
    decode sequences come first; ``jetfire_prefill_has_context`` is always set."""
    qsl = [int(x) for x in query_start_loc_cpu]
    lens = [int(x) for x in seq_lens_cpu]
    sp = split_mixed_batch(qsl, lens)
    metadata.jetfire_prefill_has_context = bool(sp.prefill_with_context)
    metadata.jetfire_max_prefill_context_len = max(
        (lens[i] - (qsl[i + 1] - qsl[i]) for i in sp.prefill_with_context), default=0)
    leading = (not sp.decode_seqs or sp.decode_seqs[0] == 0) and sp.ordered
    if leading:
        metadata.num_decodes = len(sp.decode_seqs)
        metadata.num_prefills = len(sp.prefill_seqs)
        metadata.num_decode_tokens = len(sp.decode_rows)
        metadata.num_prefill_tokens = len(sp.prefill_rows)
    return metadata


@dataclass
class MixedBatchStats:
    """Running totals (KVPoolManager.record_mixed_batch, jetfire_vllm/adapter/kv_pool.py:321-333)."""
    mixed_batch_count: int = 0
    mixed_batch_prefill_seqs: int = 0
    mixed_batch_decode_seqs: int = 0
    mixed_batch_prefill_tokens: int = 0
    mixed_batch_decode_tokens: int = 0
    handed_back: dict = field(default_factory=dict)     # reason -> count

    def record(self, *, prefill_seqs, decode_seqs, prefill_tokens, decode_tokens) -> None:
        self.mixed_batch_count += 1
        self.mixed_batch_prefill_seqs += int(prefill_seqs)
        self.mixed_batch_decode_seqs += int(decode_seqs)
        self.mixed_batch_prefill_tokens += int(prefill_tokens)
        self.mixed_batch_decode_tokens += int(decode_tokens)

    def miss(self, reason: str) -> None:
        self.handed_back[reason] = self.handed_back.get(reason, 0) + 1

    def reset(self) -> None:
        self.__init__()


MIXED_STATS = MixedBatchStats()

PrefillAttention = Callable[..., None]


def flash_varlen_prefill(*, q, k, v, out, cu_seqlens, max_seqlen, impl, layer, attn_metadata) -> None:
    """Default attention for the prefill rows: vLLM's variable-length flash attention with the
    implementation's own settings (the arguments of decode_path.py:1500-1517).  Raises
    ImportError where neither vLLM's nor the flash_attn package's function can be imported."""
    fn = _resolve_flash_varlen()
    window = getattr(impl, "sliding_window", None)
    kwargs = dict(q=q, k=k, v=v, out=out, cu_seqlens_q=cu_seqlens, cu_seqlens_k=cu_seqlens,
                  max_seqlen_q=int(max_seqlen), max_seqlen_k=int(max_seqlen),
                  softmax_scale=float(impl.scale), causal=bool(getattr(attn_metadata, "causal", True)),
                  alibi_slopes=getattr(impl, "alibi_slopes", None))
    if window is not None:
        kwargs["window_size"] = list(window) if _FLASH_FROM_VLLM else tuple(window)
    softcap = getattr(impl, "logits_soft_cap", None)
    if softcap:
        kwargs["softcap"] = softcap
    fa_version = getattr(impl, "vllm_flash_attn_version", None)
    if _FLASH_FROM_VLLM:
        if fa_version is not None:
            kwargs["fa_version"] = fa_version
        fn(**kwargs)
    else:                       # the flash_attn package returns its result
        kwargs.pop("out")
        out.copy_(fn(**kwargs))


_FLASH_FN = None
_FLASH_FROM_VLLM = False


def _resolve_flash_varlen():
    global _FLASH_FN, _FLASH_FROM_VLLM
    if _FLASH_FN is not None:
        return _FLASH_FN
    errors = []
    for module, from_vllm in (("vllm.vllm_flash_attn", True), ("flash_attn", False)):
        try:
            mod = __import__(module, fromlist=["flash_attn_varlen_func"])
            _FLASH_FN, _FLASH_FROM_VLLM = mod.flash_attn_varlen_func, from_vllm
            return _FLASH_FN
        except Exception as exc:   # the package may be present and still fail to load its kernels
            errors.append(f"{module}: {exc}")
    raise ImportError("no variable-length flash attention for the prefill rows of a mixed step ("
                      + "; ".join(errors) + "); pass prefill_attention=")


def _mixed_unsupported(*, impl, query, attn_metadata, cfg: JetFireConfig, store) -> str | None:
    """Gate in the order of try_jetfire_prefill (decode_path.py:1205-1222): a reason on a miss."""
    if not cfg.enabled:
        return "pool_disabled"
    if attn_metadata is None:
        return "profiling_run"
    if int(getattr(impl, "dcp_world_size", 1) or 1) > 1:
        return "decode_context_parallel"
    if getattr(getattr(impl, "attn_type", None), "name", "DECODER") != "DECODER":
        return "attn_type"
    if getattr(attn_metadata, "use_cascade", False):
        return "cascade"
    if int(attn_metadata.num_actual_tokens) <= 1:
        return "single_token"
    if int(attn_metadata.max_query_len) == 1:
        return "pure_decode"
    if store is None:
        return "layer_config_missing"
    if int(query.shape[-1]) != store.head_dim and int(query.shape[-1]) % store.head_dim != 0:
        return "head_dim_mismatch"
    return None


def _decode_metadata(attn_metadata, seq_lens, block_table, max_seq_len, n, device) -> SimpleNamespace:
    return SimpleNamespace(seq_lens=seq_lens, max_seq_len=int(max_seq_len), max_query_len=1,
                           num_actual_tokens=n, block_table=block_table, use_cascade=False,
                           query_start_loc=torch.arange(n + 1, device=device, dtype=torch.int32),
                           causal=getattr(attn_metadata, "causal", True),
                           max_num_splits=getattr(attn_metadata, "max_num_splits", 1))


def try_jetfire_mixed(*, impl, layer, query, key, value, attn_metadata, output, store=None,
                      cfg: JetFireConfig | None = None, prefill_attention: PrefillAttention | None = None,
                      stats: MixedBatchStats | None = None):
    """A step with both decode and prefill sequences.  Returns ``output`` when both parts were
    written, None when the step is not one this path serves (the caller then runs its native
    attention over the whole step; nothing has been written to ``output`` in that case).

    ``query (T, H_q, D)`` or ``(T, H_q * D)``, ``key`` / ``value`` likewise with the KV heads,
    ``output`` like ``query``.  The packed cache must already hold this step's tokens
    (``do_kv_cache_update`` runs before ``forward``)."""
    cfg = cfg or get_jetfire_config()
    stats = stats if stats is not None else MIXED_STATS
    reason = _mixed_unsupported(impl=impl, query=query, attn_metadata=attn_metadata, cfg=cfg, store=store)
    if reason is not None:
        stats.miss(reason)
        return None
    H_q, H_kv, D = int(layer.num_heads), int(layer.num_kv_heads), int(layer.head_size)
    if query.is_cuda and torch.cuda.is_current_stream_capturing():
        stats.miss("stream_capture")     # the decode part waits for the host correction
        return None
    counts = [getattr(attn_metadata, name, None)
              for name in ("num_decodes", "num_prefills", "num_decode_tokens", "num_prefill_tokens")]
    has_context = getattr(attn_metadata, "jetfire_prefill_has_context", None)
    ordered = all(c is not None for c in counts) and has_context is False
    if ordered:
        nd, npre, ndt, npt = (int(c) for c in counts)
        if nd == 0 or npre == 0:
            stats.miss("not_mixed")
            return None
        if ndt != nd:       # more than one query token per decode sequence (speculative decoding)
            stats.miss("multi_token_decode")
            return None
        dec_rows = slice(0, nd)
        pre_rows = slice(ndt, ndt + npt)
        cu = (attn_metadata.query_start_loc[nd:nd + npre + 1] - ndt).to(torch.int32)
        max_len = int(attn_metadata.max_query_len)
        dec_meta = _decode_metadata(attn_metadata, attn_metadata.seq_lens[:nd], attn_metadata.block_table[:nd],
                                    attn_metadata.max_seq_len, nd, query.device)
        n_dec, n_pre_seqs, n_pre_tok = nd, npre, npt
    else:
        if has_context:
            stats.miss("prefill_with_context")
            return None
        n_seqs = int(attn_metadata.seq_lens.numel())
        qsl = attn_metadata.query_start_loc[:n_seqs + 1].to("cpu", dtype=torch.int64).tolist()
        lens = attn_metadata.seq_lens.to("cpu", dtype=torch.int64).tolist()
        sp = split_mixed_batch(qsl, lens)
        if not sp.mixed:
            stats.miss("not_mixed")
            return None
        if sp.prefill_with_context:
            stats.miss("prefill_with_context")
            return None
        dev = query.device
        dec_rows = torch.tensor(sp.decode_rows, device=dev, dtype=torch.long)
        pre_rows = torch.tensor(sp.prefill_rows, device=dev, dtype=torch.long)
        cu = torch.tensor(sp.prefill_cu, device=dev, dtype=torch.int32)
        max_len = sp.max_prefill_len
        seq_idx = torch.tensor(sp.decode_seqs, device=attn_metadata.seq_lens.device, dtype=torch.long)
        sub_lens = attn_metadata.seq_lens.index_select(0, seq_idx)
        sub_bt = attn_metadata.block_table.index_select(0, seq_idx.to(attn_metadata.block_table.device))
        dec_meta = _decode_metadata(attn_metadata, sub_lens, sub_bt, max(lens[i] for i in sp.decode_seqs),
                                    len(sp.decode_seqs), dev)
        n_dec, n_pre_seqs, n_pre_tok = len(sp.decode_seqs), len(sp.prefill_seqs), len(sp.prefill_rows)

    def rows_of(t, rows, heads):
        picked = t[rows] if isinstance(rows, slice) else t.index_select(0, rows)
        return picked.reshape(picked.shape[0], heads, D)

    # decode rows first: if they cannot be served nothing has been written yet
    q_dec = rows_of(query, dec_rows, H_q).contiguous()
    out_dec = torch.empty(n_dec, H_q * D, dtype=output.dtype, device=output.device)
    done = try_jetfire_decode(impl=impl, layer=layer, query=q_dec, attn_metadata=dec_meta, output=out_dec,
                              store=store, cfg=cfg)
    if done is None:
        stats.miss("decode_part_unsupported")
        return None
    attend = prefill_attention or flash_varlen_prefill
    q_pre = rows_of(query, pre_rows, H_q)
    k_pre = rows_of(key, pre_rows, H_kv)
    v_pre = rows_of(value, pre_rows, H_kv)
    direct = isinstance(pre_rows, slice) and output.is_contiguous()
    out_pre = (output[pre_rows].view(n_pre_tok, H_q, D) if direct
               else torch.empty(n_pre_tok, H_q, D, dtype=output.dtype, device=output.device))
    attend(q=q_pre, k=k_pre, v=v_pre, out=out_pre, cu_seqlens=cu, max_seqlen=max_len, impl=impl, layer=layer,
           attn_metadata=attn_metadata)
    def write_back(rows, src):
        src = src.reshape(src.shape[0], *output.shape[1:])
        if isinstance(rows, slice):
            output[rows].copy_(src)
        else:
            output.index_copy_(0, rows, src)

    write_back(dec_rows, out_dec)
    if not direct:
        write_back(pre_rows, out_pre)
    stats.record(prefill_seqs=n_pre_seqs, decode_seqs=n_dec, prefill_tokens=n_pre_tok, decode_tokens=n_dec)
    return output
