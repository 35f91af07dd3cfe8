"""Which options of the objective go together.

``check_options`` is called once at the top of ``scan.loss_fn`` with the loss configuration (after the GDN memory has switched the
write off), the model configuration and a predicate telling whether the parameter tree has a given leaf.  Every rule is a pair
(the combination is refused when the condition holds, what to tell the user); the combinations refused are those the reference
refuses (src/ttt/chunk_scan.py:300-470), stated here as one table instead of checks scattered through the scan.
"""
from __future__ import annotations

from typing import Callable, List, Tuple


def _rules(cfg, mc, has_leaf: Callable[[str], bool], use_gdn: bool, gdn_requested: dict) -> List[Tuple[bool, str]]:
    one_view = cfg.inner_views == 1
    has_inner = not (cfg.no_write or cfg.inner_from_outer)
    plain_causal = cfg.inner_task == "causal" and one_view and has_inner and not cfg.write_off
    schemes = not cfg.write.plain
    rules = [
        (use_gdn and any(gdn_requested.values()),
         "a GDN memory has no inner stream, so these do not apply: " + ", ".join(k for k, v in gdn_requested.items() if v)),
        (cfg.outer_views < 1, "outer_views must be at least 1"),
        (cfg.outer_views > 1 and bool(cfg.distill or cfg.mtp or cfg.reread_chunks or cfg.inner_from_outer or cfg.per_sequence
                                      or cfg.per_token or mc.read_block),
         "several outer views are for training only: not with distill, mtp, reread_chunks, inner_from_outer, per-sequence / "
         "per-token scores or read_block"),
        (bool(cfg.mtp or cfg.distill) and (not has_inner or cfg.inner_task == "split" or not one_view),
         "distill and mtp need a write with one view under the mask or causal task"),
        (cfg.write_off and (not has_inner or bool(cfg.distill or cfg.mtp) or not one_view or cfg.inner_feat != "off"),
         "write_off keeps exactly one plain inner stream: not with no_write, inner_from_outer, distill, mtp, views or inner_feat"),
        (cfg.aux_causal_weight > 0 and not has_inner, "aux_causal_weight needs an inner stream"),
        (bool(cfg.write_plan) and (schemes or not plain_causal or bool(cfg.reread_chunks) or min(cfg.write_plan or (0,)) < 0),
         "write_plan needs the plain causal write (one view, a write, no re-read) and non-negative step counts"),
        (schemes and (not plain_causal or bool(cfg.distill or cfg.mtp) or cfg.inner_feat != "off" or cfg.inner_update_frac < 1.0),
         "the write schemes build on the plain causal write: one view, a write, and none of write_off, distill, mtp, inner_feat, "
         "inner_update_frac"),
        (schemes and cfg.write.kvb_weight > 0 and not has_leaf("inner_kvb_value.weight"),
         "inner_kvb_weight needs a model built with inner_kvb_head"),
        (cfg.self_prior > 0 and (use_gdn or not has_inner or cfg.write_off or bool(cfg.write_plan) or bool(cfg.reread_chunks) or not one_view),
         "self_prior reads a chunk after its own write, which needs a fast-weight write with one view and no write plan or re-read"),
        (cfg.mtp and (not cfg.outer_shift or cfg.inner_task != "causal"), "mtp needs outer_shift and the causal write"),
        (cfg.mtp and not has_leaf("mtp_head.weight"), "mtp needs a model built with mtp_head"),
        (bool(cfg.reread_chunks) and (cfg.segment_chunks <= 0 or cfg.reread_chunks % max(cfg.segment_chunks, 1) != 0),
         "reread_chunks needs segment_chunks > 0 that divides it (the window restarts at a segment boundary)"),
        (bool(cfg.reread_chunks) and cfg.distill, "reread_chunks cannot be combined with distill"),
        (cfg.inner_feat != "off" and not has_inner, "inner_feat needs the inner stream"),
        (cfg.inner_feat != "off" and has_inner and not has_leaf("inner_feat_head.weight"), "inner_feat needs a model built with inner_feat_head"),
        (bool(mc.read_block) and cfg.distill, "read_block has no distillation teacher stream"),
    ]
    return rules


def check_options(cfg, mc, has_leaf: Callable[[str], bool], use_gdn: bool = False, gdn_requested: dict = None) -> None:
    """Raise ``ValueError`` for the first refused combination.  With a non-plain write its own parameters are checked too."""
    if not cfg.write.plain:
        cfg.write.check(mc.chunk_size)
    for refused, why in _rules(cfg, mc, has_leaf, use_gdn, gdn_requested or {}):
        if refused:
            raise ValueError(why)


def check_geometry(seq_len: int, mc, segment_chunks: int, n_chunks: int) -> int:
    """Chunks per segment for a sequence of ``n_chunks`` chunks (re-read chunks included); refuses lengths that do not tile."""
    if seq_len % mc.chunk_size:
        raise ValueError(f"seq_len {seq_len} not a multiple of chunk_size {mc.chunk_size}")
    per_segment = segment_chunks or n_chunks
    if n_chunks % per_segment:
        raise ValueError(f"{n_chunks} chunks not a multiple of segment_chunks {per_segment}")
    if per_segment < mc.window_chunks and per_segment < n_chunks:
        raise ValueError(f"segment_chunks {per_segment} < window_chunks {mc.window_chunks}: the carried window would be short")
    return per_segment
