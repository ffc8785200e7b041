"""TEST INFRASTRUCTURE — CPU restatement of the reference's attention math.  Not a product path:
only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import it.

Restates, in independent code, what FlashAttention v2.3.3 uses as ground truth for its kernels:

  * attention_oracle  <- attention_ref            tests/test_flash_attn.py:183-259
  * visibility_mask   <- construct_local_mask     tests/test_flash_attn.py:153-180
  * lse_oracle        <- kernel LSE semantics     csrc/flash_attn/src/flash_fwd_kernel.h:505-516
                                                  (no reference test compares LSE; same convention as
                                                  normalize_flash_attn_S, tests/test_flash_attn.py:470-476)
  * rotary_oracle     <- apply_rotary_emb_torch   flash_attn/layers/rotary.py:11-32 with the position
                                                  gather of index_cos_sin, tests/test_rotary.py:32-42
  * kvcache_oracle    <- expected cache/out state tests/test_flash_attn.py:1758-1842
  * merge_oracle      <- split-KV combine math    csrc/flash_attn/src/flash_fwd_kernel.h:1227-1298

Pinned: tests/test_oracle.py checks every function against tests/golden/reference_cases.pt, which
tests/golden/make_golden.py produced by running the reference's own functions (loaded from the
reference tree by AST extraction) on seeded inputs.
"""
import math

import torch


def visibility_mask(seqlen_q, seqlen_k, window=(-1, -1), q_lens=None, k_lens=None, device=None):
    """Boolean (.., seqlen_q, seqlen_k), True where key j is visible to query i.

    Rule (bottom-right aligned): i + sk - sq - window[0] <= j <= i + sk - sq + window[1] and j < sk,
    with a negative window side unbounded; sk / sq are per-batch lengths when given (shape (B,)).
    Returned shape is (seqlen_q, seqlen_k) without lengths, else (B, 1, seqlen_q, seqlen_k).
    """
    i = torch.arange(seqlen_q, device=device).view(-1, 1)
    j = torch.arange(seqlen_k, device=device).view(1, -1)
    if q_lens is None and k_lens is None:
        sq, sk = seqlen_q, seqlen_k
    else:
        sq = seqlen_q if q_lens is None else q_lens.view(-1, 1, 1, 1).to(torch.long)
        sk = seqlen_k if k_lens is None else k_lens.view(-1, 1, 1, 1).to(torch.long)
    diag = i + (sk - sq)
    vis = (j < sk) if torch.is_tensor(sk) else (j < sk).expand(seqlen_q, seqlen_k).clone()
    if window[1] >= 0:
        vis = vis & (j <= diag + window[1])
    if window[0] >= 0:
        vis = vis & (j >= diag - window[0])
    return vis


def _expand_kv(x, heads):
    g = heads // x.shape[2]
    return x if g == 1 else x.repeat_interleave(g, dim=2)


def attention_oracle(q, k, v, query_padding_mask=None, key_padding_mask=None, dropout_p=0.0, dropout_mask=None,
                     causal=False, window_size=(-1, -1), upcast=True, reorder_ops=False):
    """out (B, Sq, H, D) and the pre-dropout softmax (B, H, Sq, Sk), both cast back to q's dtype.

    upcast=True computes in fp32 (the truth); upcast=False with reorder_ops=True computes in the
    input dtype with the scale applied to k (the error yardstick of the reference's tests).
    """
    if causal:
        window_size = (window_size[0], 0)
    in_dtype = q.dtype
    if upcast:
        q, k, v = q.float(), k.float(), v.float()
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    k, v = _expand_kv(k, H), _expand_kv(v, H)
    inv = math.sqrt(D)
    qs, ks = (q, k / inv) if reorder_ops else (q / inv, k)
    scores = torch.matmul(qs.permute(0, 2, 1, 3), ks.permute(0, 2, 3, 1))  # (B, H, Sq, Sk)
    neg = float("-inf")
    if key_padding_mask is not None:
        scores = scores.masked_fill(~key_padding_mask.view(B, 1, 1, Sk), neg)
    windowed = window_size[0] >= 0 or window_size[1] >= 0
    if windowed:
        q_lens = None if query_padding_mask is None else query_padding_mask.sum(-1)
        k_lens = None if key_padding_mask is None else key_padding_mask.sum(-1)
        # the reference bounds the right edge by min(diag + w1, sk), i.e. it lets j == sk through;
        # key padding (applied above) is what removes j >= sk (tests/test_flash_attn.py:170-180)
        hidden = _window_hidden(Sq, Sk, window_size, q_lens, k_lens, q.device)
        scores = scores.masked_fill(hidden, neg)
        hidden_rows = hidden.all(dim=-1, keepdim=True)
    probs = torch.softmax(scores, dim=-1)
    if windowed:
        probs = probs.masked_fill(hidden_rows, 0.0)
    if query_padding_mask is not None:
        probs = probs.masked_fill(~query_padding_mask.view(B, 1, Sq, 1), 0.0)
    kept = probs if dropout_mask is None else probs.masked_fill(~dropout_mask, 0.0)
    out = torch.matmul(kept, (v * (1.0 / (1.0 - dropout_p))).permute(0, 2, 1, 3)).permute(0, 2, 1, 3)
    if query_padding_mask is not None:
        out = out.masked_fill(~query_padding_mask.view(B, Sq, 1, 1), 0.0)
    return out.to(in_dtype), probs.to(in_dtype)


def _window_hidden(Sq, Sk, window, q_lens, k_lens, device):
    """True where the reference's construct_local_mask masks (tests/test_flash_attn.py:153-180)."""
    i = torch.arange(Sq, device=device).view(-1, 1)
    j = torch.arange(Sk, device=device).view(1, -1)
    sk = Sk if k_lens is None else k_lens.view(-1, 1, 1, 1).to(torch.long)
    sq = Sq if q_lens is None else q_lens.view(-1, 1, 1, 1).to(torch.long)
    diag = i + (sk - sq)
    if window[0] < 0:
        return j > diag + window[1]
    right = diag + window[1]
    right = torch.minimum(right, sk if torch.is_tensor(sk) else torch.full_like(right, sk))
    return (j > right) | (j < diag - window[0])


def lse_oracle(q, k, key_padding_mask=None, query_padding_mask=None, causal=False, window_size=(-1, -1),
               softmax_scale=None):
    """fp32 (B, H, Sq): ln sum_j exp(scale * q_i.k_j) over visible keys, +inf where none is visible."""
    if causal:
        window_size = (window_size[0], 0)
    q, k = q.float(), k.float()
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    k = _expand_kv(k, H)
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    scores = torch.matmul(q.permute(0, 2, 1, 3), k.permute(0, 2, 3, 1)) * scale
    q_lens = None if query_padding_mask is None else query_padding_mask.sum(-1)
    k_lens = None if key_padding_mask is None else key_padding_mask.sum(-1)
    vis = visibility_mask(Sq, Sk, window_size, q_lens, k_lens, q.device)
    scores = scores.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    return torch.where(torch.isinf(lse) & (lse < 0), torch.full_like(lse, float("inf")), lse)


def rotary_oracle(x, cos, sin, seqlen_offsets=0, interleaved=False):
    """Rotary embedding of x (B, S, H, D) with table rows seqlen_offsets[b] + s.

    cos/sin: (seqlen_ro, rotary_dim/2).  Non-interleaved pairs dim i with i + rotary_dim/2
    (GPT-NeoX), interleaved pairs 2i with 2i+1.  Computed in x's dtype like the torch reference.
    """
    B, S, H, D = x.shape
    half = cos.shape[-1]
    rd = 2 * half
    if torch.is_tensor(seqlen_offsets):
        pos = seqlen_offsets.view(B, 1).to(torch.long) + torch.arange(S, device=x.device).view(1, S)
    else:
        pos = (torch.arange(S, device=x.device) + int(seqlen_offsets)).view(1, S).expand(B, S)
    c = cos[pos].unsqueeze(2)  # (B, S, 1, half)
    s = sin[pos].unsqueeze(2)
    xr = x[..., :rd]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        rot = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        a, b = xr[..., :half], xr[..., half:]
        rot = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return torch.cat((rot.to(x.dtype), x[..., rd:]), dim=-1)


def kvcache_oracle(q, k_cache, v_cache, k_new=None, v_new=None, cos=None, sin=None, cache_seqlens=None,
                   cache_batch_idx=None, causal=False, window_size=(-1, -1), rotary_interleaved=True, upcast=True,
                   reorder_ops=False):
    """Expected (out, k_cache_after, v_cache_after) of flash_attn_with_kvcache.

    The cache tensors returned are the rows selected by cache_batch_idx (all rows when None), with
    the new keys (rotated at cache_seqlens[b] + i) and values written at [cache_seqlens[b], +seqlen_new).
    q is rotated at cache_seqlens[b] + i when causal/windowed, at cache_seqlens[b] otherwise.
    """
    B, Sq, H, D = q.shape
    Sk = k_cache.shape[1]
    Hk = k_cache.shape[2]
    local = window_size[0] >= 0 or window_size[1] >= 0
    if cache_seqlens is None:
        cache_seqlens = torch.full((B,), Sk, dtype=torch.int32, device=q.device)
    sel = slice(None) if cache_batch_idx is None else cache_batch_idx.to(torch.long)
    kc, vc = k_cache[sel].clone(), v_cache[sel].clone()
    q_r, k_r = q, k_new
    if cos is not None:
        if causal or local:
            q_r = rotary_oracle(q, cos, sin, cache_seqlens, rotary_interleaved)
        else:
            flat = q.reshape(B, 1, Sq * H, D)
            q_r = rotary_oracle(flat, cos, sin, cache_seqlens, rotary_interleaved).reshape(B, Sq, H, D)
        k_r = rotary_oracle(k_new, cos, sin, cache_seqlens, rotary_interleaved)
    n_new = 0
    if k_new is not None:
        n_new = k_new.shape[1]
        for b in range(B):
            s0 = int(cache_seqlens[b])
            kc[b, s0:s0 + n_new] = k_r[b]
            vc[b, s0:s0 + n_new] = v_new[b]
    key_mask = torch.arange(Sk, device=q.device).view(1, Sk) < (cache_seqlens.view(B, 1).to(torch.long) + n_new)
    out, _ = attention_oracle(q_r, kc, vc, None, key_mask, 0.0, None, causal=causal, window_size=window_size,
                              upcast=upcast, reorder_ops=reorder_ops)
    return out, kc, vc


def merge_oracle(out_parts, lse_parts):
    """Combine partial attention outputs (P, rows, D) with their LSEs (P, rows): LSE = logsumexp_p,
    out = sum_p exp(lse_p - LSE) out_p; rows whose parts are all -inf give out 0 and LSE +inf."""
    lse = torch.logsumexp(lse_parts.float(), dim=0)
    w = torch.exp(lse_parts.float() - lse.unsqueeze(0))
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    out = (w.unsqueeze(-1) * out_parts.float()).sum(0)
    lse = torch.where(torch.isinf(lse) & (lse < 0), torch.full_like(lse, float("inf")), lse)
    return out, lse
