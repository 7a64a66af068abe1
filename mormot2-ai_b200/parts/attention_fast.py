"""The tensor-core attention kernels of the bfloat16 path (``csrc/attention_mma.cu``): which
kernel takes a call, and how a sequence's pages are shared out over CTAs."""
from __future__ import annotations


import torch

from .. import kernels as K
from ..cache.pages import pages_for

FAST_HEAD_DIMS = (64, 128)
MAX_DECODE_SPLITS = 8       # the splits of a sequence are one thread-block cluster


def decode_splits(line, T: int, nh: int, nkv: int, sms: int, window: int,
                  keep_first: int = 0) -> int:
    """Over how many CTAs the pages of a sequence are dealt out in a decode step of T tokens.
    Every CTA pays a fixed price (index loads before its first key, the merge at its end), so
    few, long CTAs win: as many as give one round of two CTAs per SM, at most 8 (the splits of a
    sequence form a thread-block cluster that merges through shared memory, and beyond that the
    merge costs more than the shorter CTAs save: measured at batch 1),
    and no more than the most pages that a sequence can hold in this line (the lengths of the
    moment do not count: a captured launch must stay valid as sequences grow)."""
    pages = line.max_pages
    if window > 0:      # the window's pages and those of positions that it never loses
        pages = min(pages, pages_for(window) + 1 + (pages_for(keep_first) if keep_first else 0))
    subs = (nh // nkv + 15) // 16
    groups = max(1, T * nkv * subs)
    return max(1, min((2 * sms) // groups, pages, MAX_DECODE_SPLITS))


MANY_SPLITS_MOST = 32       # CTAs that share one long sequence through scratch memory, at most


def decode_many_splits(step, nh: int, nkv: int, sms: int) -> int:
    """A batch so small that even eight splits a sequence leave SMs idle (one or two sequences
    at eight KV heads) whose longest sequence is long (``step.long``): a cluster's eight CTAs at
    ≈ 50 GB/s each then stream it at less than half the memory's rate. Returns how many CTAs
    share a sequence's pages through scratch memory and a second kernel that adds them up
    (about one CTA per SM), or 0 where the cluster form serves. The engine captures passes
    with ``step.long`` as graphs of their own, so the choice may depend on it."""
    subs = (nh // nkv + 15) // 16
    groups = max(1, step.T * nkv * subs)
    if not step.long or groups * MAX_DECODE_SPLITS > sms:
        return 0
    return min(sms // groups, MANY_SPLITS_MOST)


def run(rt, q, q_stride, out, step, line, nh, nkv, hd, window, scale, sink=None,
        softcap: float = 0.0, gate=None, gate_stride: int = 0, slopes=None,
        keep_first: int = 0) -> bool:
    """True if a fast kernel took the call; False: the caller uses the general kernel.
    ``sink``: float32 [nh], one more term exp(sink[h]) in every softmax denominator.
    ``softcap`` > 0: scores become softcap * tanh(score / softcap); ``gate``: bfloat16 logits,
    head h of token t at ``gate[t * gate_stride + h]``, whose sigmoid multiplies the head's
    output. ``slopes`` (float32 [nh], a bias slopes[h] * distance taken off the scores) and
    ``keep_first`` (positions at a sequence's start that a window never loses) are served by
    the ``mma.sync`` kernels; the tcgen05 prefill kernel does not take them."""
    if hd not in FAST_HEAD_DIMS or q.dtype != torch.bfloat16 or q_stride % 8 or q.data_ptr() % 16:
        return False
    if scale <= 0 or (gate is not None and gate.dtype != torch.bfloat16):
        return False
    more = (softcap, gate, gate_stride, slopes, keep_first)
    plain_mask = slopes is None and not keep_first
    if step.decode:
        many = decode_many_splits(step, nh, nkv, rt.sms) if window == 0 else 0
        if many > MAX_DECODE_SPLITS and step.T * nh * many * (hd + 2) <= rt.attention_scratch.numel():
            K.attention_decode(q, q_stride, out, step, line, nh, nkv, hd, window, scale, many,
                               rt.attention_scratch, rt.error_word, sink, *more)
            return True
        splits = decode_splits(line, step.T, nh, nkv, rt.sms, window, keep_first)
        K.attention_decode_clusters(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                                    splits, rt.error_word, sink, *more)
        return True
    if out.stride(0) % 8 or out.data_ptr() % 16:
        return False
    if hd == 128 and q.stride(1) == 1 and plain_mask:
        # S and O in tensor memory, tiles by TMA (csrc/attention_tc.cu)
        K.attention_prefill_tc(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                               rt.error_word, sink, softcap, gate, gate_stride)
        return True
    K.attention_prefill(q, q_stride, out, step, line, nh, nkv, hd, window, scale,
                        rt.error_word, sink, *more)
    return True
