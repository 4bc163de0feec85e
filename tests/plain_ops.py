"""Plain float32 restatements of every kernel, one function per kernel, written as loops
over sequences and tokens from the reference's formulas.  They have the signatures of
``vapi_b200.ops`` so that (a) each CUDA kernel can be compared with its plain version alone
and (b) the host side of the engine (cache manager, packer, step function, scheduler) can be
exercised on a CPU by standing these in for the kernels.  They are test code: nothing in the
package imports them, and the package has no CPU path of its own.
"""
from __future__ import annotations

import math

import torch


def _f(t):
    return t.to(torch.float32)


def embed(table, tokens, status=None, next_weight=None, scale=1.0):
    out = _f(table[tokens.long()]) * torch.tensor(scale, dtype=torch.float32)
    if next_weight is None:
        return out
    return out, (out ** 2).sum(1)[None, :], (out * next_weight).to(torch.bfloat16)


def resolve_tokens(tokens, src, prev, status=None):
    """tokens[i] = prev[src[i]] where src[i] >= 0 (tokens the step before sampled on the device)."""
    m = src >= 0
    tokens[m] = prev[src[m].long()]


def add_residual_ss(x, delta, next_weight):
    x += _f(delta)
    return (x ** 2).sum(1)[None, :], (x * next_weight).to(torch.bfloat16)


def skinny_applies(rows, weight):
    return False


def tc_applies(rows, weight):
    return False


def few_rows_applies(rows, weight):
    return False


def add_rmsnorm(x, delta, weight, eps, out_dtype, rows=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:633-648: residual add, then RMSNorm."""
    if rows is None:
        if delta is not None:
            x += _f(delta)
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + _f(delta[rows.long()])
    y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight
    return y.to(out_dtype)


def add_residual(x, delta):
    x += _f(delta)


def swiglu(g):
    """crates/vapi-backend-candle/src/fused.rs:157-165."""
    f = g.shape[1] // 2
    a, b = _f(g[:, :f]), _f(g[:, f:])
    return ((a / (1.0 + torch.exp(-a))) * b).to(g.dtype)


def linear(x, weight, bias=None, out_dtype=None):
    y = _f(x) @ _f(weight).t()
    if bias is not None:
        y = y + _f(bias)
    return y.to(out_dtype or x.dtype)


def strict_fp32():
    pass


def rope_cos_sin(positions, inv_freq):
    """crates/vapi-backend-candle/src/models/lfm2.rs:169-178: angle = p as f32 * inv_freq."""
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def qk_norm_rope_write(qkv, nh, nkv, d, q_weight, k_weight, eps, cos, sin, rot, cache_layer,
                       slot_mapping, status=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:364-375."""
    n = qkv.shape[0]
    heads = qkv.view(n, nh + 2 * nkv, d)
    page = cache_layer.shape[3] if cache_layer is not None else 0
    for t in range(n):
        for h in range(nh + 2 * nkv):
            v = _f(heads[t, h])
            is_q, is_k = h < nh, nh <= h < nh + nkv
            w = q_weight if is_q else (k_weight if is_k else None)
            if w is not None:
                v = v * torch.rsqrt(v.pow(2).mean() + eps) * w
            if (is_q or is_k) and cos is not None:
                half = rot // 2
                a, b = v[:half].clone(), v[half:rot].clone()
                v = v.clone()
                v[:half] = a * cos[t] - b * sin[t]
                v[half:rot] = b * cos[t] + a * sin[t]
            if is_q:
                heads[t, h] = v.to(qkv.dtype)
            elif cache_layer is not None:
                slot = int(slot_mapping[t])
                g = h - nh if is_k else h - nh - nkv
                cache_layer[slot // page, 0 if is_k else 1, g, slot % page] = v.to(cache_layer.dtype)


def attention_splits(num_seqs, max_q, max_k, nh, nkv):
    return 1


def paged_attention(q, q_row_stride, cache_layer, block_table, cu_q, seqlens_k, n, num_seqs, max_q,
                    max_k, nh, nkv, d, scale, window=0, splits=None, status=None):
    """crates/vapi-backend-candle/src/attention.rs:90-163: gather each sequence's keys
    through its block table; query j of len_q over len_k keys sits at len_k - len_q + j and
    sees keys i <= its position (and i > position - window)."""
    page = cache_layer.shape[3]
    rep = nh // nkv
    qh = q.reshape(n, -1)[:, :nh * d].reshape(n, nh, d)
    out = torch.zeros((n, nh * d), dtype=torch.float32)
    for s in range(num_seqs):
        q0, q1, klen = int(cu_q[s]), int(cu_q[s + 1]), int(seqlens_k[s])
        qlen = q1 - q0
        keys = torch.zeros((klen, nkv, d))
        vals = torch.zeros((klen, nkv, d))
        lo_needed = 0 if window <= 0 else max(0, klen - qlen - window + 1)
        for i in range(lo_needed, klen):
            pg = int(block_table[s, i // page])
            keys[i] = _f(cache_layer[pg, 0, :, i % page])
            vals[i] = _f(cache_layer[pg, 1, :, i % page])
        for j in range(qlen):
            p = klen - qlen + j
            lo = 0 if window <= 0 else max(0, p - window + 1)
            for h in range(nh):
                g = h // rep
                sc = (keys[lo:p + 1, g] @ _f(qh[q0 + j, h])) * scale
                pr = torch.softmax(sc, 0)
                out[q0 + j, h * d:(h + 1) * d] = pr @ vals[lo:p + 1, g]
    return out.to(q.dtype)


def shortconv(h3, in_bias, taps, conv_bias, state_layer, state_slots, tok_seq, cu_q, positions, status=None):
    """crates/vapi-backend-candle/src/models/lfm2.rs:509-565 with the state kept as the last
    L-1 rows of g per request instead of paged rows: per sequence, rebuild the history from
    the state, run the causal conv over the portion, store the new last L-1 rows."""
    n, H, L = h3.shape[0], h3.shape[1] // 3, taps.shape[0]
    dt = h3.dtype
    out = torch.zeros((n, H), dtype=torch.float32)
    S = cu_q.numel() - 1
    for s in range(S):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        p0 = int(positions[r0])
        slot = int(state_slots[s])
        hist = []                                   # g at positions p0-(L-1) .. p0-1
        for j in range(L - 1):
            pos = p0 - (L - 1) + j
            hist.append(_f(state_layer[slot, j]) if pos >= 0 else torch.zeros(H))
        for r in range(r0, r1):
            B, C, x = _f(h3[r, :H]), _f(h3[r, H:2 * H]), _f(h3[r, 2 * H:])
            if in_bias is not None:
                B, C, x = B + in_bias[:H], C + in_bias[H:2 * H], x + in_bias[2 * H:]
            g = (B * x).to(dt).to(torch.float32)    # the stored row has the storage precision
            hist.append(g)
            acc = torch.zeros(H)
            for k in range(L):
                acc = acc + taps[k] * hist[len(hist) - L + k]
            if conv_bias is not None:
                acc = acc + conv_bias
            out[r] = C * acc
            hist = hist[-(L - 1):] if L > 1 else []
        for j in range(L - 1):
            state_layer[slot, j] = hist[j].to(dt)
    return out.to(dt)


def _mix64(x):
    m = (1 << 64) - 1
    x ^= x >> 33
    x = (x * 0xff51afd7ed558ccd) & m
    x ^= x >> 33
    x = (x * 0xc4ceb9fe1a85ec53) & m
    x ^= x >> 33
    return x


def gumbel_noise(seed, draw, vocab):
    """crates/vapi-backend-candle/src/fused.rs:252-293."""
    m = (1 << 64) - 1
    key = _mix64((seed ^ _mix64((draw + 0x9E3779B97F4A7C15) & m)) & m)
    out = torch.empty(vocab, dtype=torch.float64)
    for v in range(vocab):
        h = _mix64((key + v * 0xBF58476D1CE4E5B9) & m)
        u = ((h >> 40) + 0.5) / 16777216.0
        out[v] = -math.log(-math.log(u))
    return out


def sample_rows(logits, mode=None, inv_t=None, seeds=None, draws=None, out=None):
    rows, vocab = logits.shape
    res = torch.zeros(rows, dtype=torch.int32) if out is None else out
    for r in range(rows):
        md = 1 if mode is None else int(mode[r])
        if md == 0:
            continue
        if md == 1:
            res[r] = int(torch.argmax(logits[r]))
        else:
            g = gumbel_noise(int(seeds[r]) & ((1 << 64) - 1), int(draws[r]), vocab)
            res[r] = int(torch.argmax(logits[r].double() * float(inv_t[r]) + g))
    return res


def sample_truncated(logits, inv_t, top_k, top_p, min_p, seeds, draws, out=None, check=False):
    """Gumbel-max over the host sampler's survivors; rows with a negative top_k are left alone."""
    rows, vocab = logits.shape
    res = torch.zeros(rows, dtype=torch.int32) if out is None else out
    for r in range(rows):
        k = int(top_k[r]) if top_k is not None else 0
        if k < 0:
            continue
        ids, _, scaled = truncated_survivors(logits[r].float().numpy(), float(inv_t[r]), k or None,
                                             float(top_p[r]) if top_p is not None else 1.0,
                                             float(min_p[r]) if min_p is not None else 0.0)
        g = gumbel_noise(int(seeds[r]) & ((1 << 64) - 1), int(draws[r]), vocab)
        best = max(ids.tolist(), key=lambda t: (float(scaled[t]) + float(g[t]), -t))
        res[r] = best
    return res


def truncated_survivors(row, inv_t, top_k=None, top_p=1.0, min_p=0.0):
    """Token ids that survive the host sampler's cuts, in its order (probability descending, then
    id), and their probabilities over the 30-nat window
    (crates/vapi-engine/src/sampler.rs:302-376): window, top-k, min-p, top-p."""
    import numpy as np
    scaled = row.astype(np.float32) * np.float32(inv_t)
    mx = scaled.max()
    keep = np.nonzero(scaled >= mx - np.float32(30.0))[0]
    e = np.exp((scaled[keep] - mx).astype(np.float64))
    prob = e / e.sum()
    order = np.lexsort((keep, -prob))
    ids, prob = keep[order], prob[order]
    if top_k:
        ids, prob = ids[:top_k], prob[:top_k]
    if min_p > 0.0:
        n = max(int(np.sum(np.cumprod(prob >= min_p * prob[0]))), 1)
        ids, prob = ids[:n], prob[:n]
    if top_p < 1.0:
        cum = np.cumsum(prob)
        n = max(min(int(np.searchsorted(cum, top_p, side="left")) + 1, len(prob)), 1)
        ids, prob = ids[:n], prob[:n]
    return ids, prob, scaled


def apply_penalties(logits, rows, toks, counts, rep, freq, pres):
    """crates/vapi-engine/src/sampler.rs:262-283."""
    for i in range(rows.numel()):
        r, t = int(rows[i]), int(toks[i])
        v = float(logits[r, t])
        p = float(rep[r])
        if p != 1.0:
            v = v / p if v > 0 else v * p
        v -= float(freq[r]) * float(counts[i])
        if float(counts[i]) > 0:
            v -= float(pres[r])
        logits[r, t] = v


# ---- blocks with norms on both sides, scaled rotary tables, general attention, recurrent mixers -----
def postnorm_add_rmsnorm(x, y, post_weight, post_eps, mult, weight, eps, out_dtype, rows=None, copy=False, branches=None):
    """x += mult * rms(y) * post_weight;  out = rms(x) * weight, or x itself with `copy` (for `rows` only, x untouched).
    branches = (y2, wa, wb, eps_b, scale): scale * (rms(y) * wa + rms(y2) * wb) stands for y."""
    add = None
    if y is not None:
        yf = _f(y)
        if branches is not None:
            y2, wa, wb, eps_b, scale = branches
            y2f = _f(y2)
            yf = scale * (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + eps_b) * wa
                          + y2f * torch.rsqrt(y2f.pow(2).mean(-1, keepdim=True) + eps_b) * wb)
        add = mult * (yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + post_eps) * post_weight)
    if rows is None:
        if add is not None:
            x += add
        src = x
    else:
        src = x[rows.long()] + (add[rows.long()] if add is not None else 0.0)
    if weight is None:
        return src.to(out_dtype) if copy else None
    return (src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out_dtype)


def scaled_add_rmsnorm(x, y1, s1, y2, s2, weight, eps, out_dtype, rows=None, copy=False, out=None):
    """x += s1 * y1 + s2 * y2 (a missing scale counts as one); out = rms(x) * weight, or x itself with `copy`; for `rows`
    only those rows and x untouched.  A given `out` is filled and returned."""
    add = None
    for y, sc in ((y1, s1), (y2, s2)):
        if y is not None:
            term = _f(y) * (sc if sc is not None else 1.0)
            add = term if add is None else add + term
    if rows is None:
        if add is not None:
            x += add
        src = x
    else:
        src = x[rows.long()] + (add[rows.long()] if add is not None else 0.0)
    if weight is None and not copy:
        return None
    res = src if weight is None else src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight
    if out is not None:
        out.copy_(res.to(out_dtype))
        return out
    return res.to(out_dtype)


def _rotate_half(v, cos_t, sin_t, rot):
    half = rot // 2
    r = v.clone()
    for i in range(half):
        r[..., i] = v[..., i] * cos_t[i] - v[..., i + half] * sin_t[i]
        r[..., i + half] = v[..., i + half] * cos_t[i] + v[..., i] * sin_t[i]
    return r


def latent_prepare(down, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, cos, sin, rot, cache_layer, page_size,
                   slot_mapping, out_dtype, status=None):
    """down [n, q_rank | kv_rank | rot_dim] float32: the query latent normed; latent normed | key part rotated, into the page."""
    n = down.shape[0]
    cq = None
    if q_rank > 0:
        a = down[:, :q_rank]
        cq = (a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps) * q_weight).to(out_dtype)
    if cache_layer is not None:
        width = kv_rank + rot_dim
        for t in range(n):
            c = down[t, q_rank:q_rank + kv_rank]
            c = c * torch.rsqrt(c.pow(2).mean() + eps) * kv_weight
            kr = down[t, q_rank + kv_rank:q_rank + width]
            if rot > 0:
                kr = _rotate_half(kr, cos[t], sin[t], rot)
            slot = int(slot_mapping[t])
            pg, off = slot // page_size, slot % page_size
            cache_layer[pg, off * width:(off + 1) * width] = torch.cat([c, kr]).to(cache_layer.dtype)
    return cq


def latent_rotate_q(q, qfull, heads, dim, rot_dim, kv_rank, cos, sin, rot):
    n = q.shape[0]
    q3 = _f(q).view(n, heads, dim + rot_dim)
    for t in range(n):
        part = q3[t, :, dim:]
        if rot > 0:
            part = _rotate_half(part, cos[t], sin[t], rot)
        qfull[t, :, kv_rank:] = part.to(qfull.dtype)


def head_products(x, w, out=None):
    """out[t, h] = x[t, h] @ w[h]"""
    res = torch.einsum("thk,hkm->thm", _f(x), _f(w)).to(x.dtype).contiguous()
    if out is None:
        return res
    out.copy_(res)
    return out


def latent_attention(q, cache_layer, page_size, block_table, cu_q, seqlens_k, n, num_seqs, max_q, max_k, heads, kv_rank, rot_dim,
                     scale, *, splits=None, status=None):
    width = kv_rank + rot_dim
    return masked_attention(q, heads * width, cache_layer, page_size, block_table, cu_q, seqlens_k, n, num_seqs, max_q, max_k,
                            heads, 1, width, kv_rank, scale, shared_kv=True)


def gated_group_rmsnorm(y, z, weight, eps, group, gate_first, out_dtype, gate="silu"):
    n, width = y.shape
    zf = _f(z)
    gate = torch.sigmoid(zf) if gate == "sigmoid" else zf / (1.0 + torch.exp(-zf))
    w = weight.repeat(width // weight.numel())
    v = y * gate if gate_first else y
    v = v.view(n, width // group, group)
    v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).view(n, width) * w
    return (v if gate_first else v * gate).to(out_dtype)


def scale_rows(x, factor):
    x *= factor
    return x


def rope_cos_sin_scaled(positions, freq, mult):
    ang = positions.to(torch.float32)[:, None] * freq[None, :]
    return torch.cos(ang) * mult, torch.sin(ang) * mult


def qk_norm_rope_write_split(qkv, nh, nkv, dk, dv, q_weight, k_weight, eps, cos, sin, rot, interleaved, cache_layer,
                             page_size, slot_mapping, status=None, whole=False, positions=None, q_temp=None):
    n = qkv.shape[0]
    for t in range(n):
        q_mult = 1.0
        if q_temp is not None:      # the query at position p times 1 + coef * ln(floor((p + 1) / every) + 1)
            q_mult = 1.0 + q_temp[0] * torch.log(torch.tensor(float((int(positions[t]) + 1) // q_temp[1] + 1), dtype=torch.float32))
        if whole:
            inv_q = torch.rsqrt(_f(qkv[t, :nh * dk]).pow(2).mean() + eps)
            inv_k = torch.rsqrt(_f(qkv[t, nh * dk:(nh + nkv) * dk]).pow(2).mean() + eps)
        for h in range(nh + 2 * nkv):
            is_q, is_k = h < nh, nh <= h < nh + nkv
            if is_q or is_k:
                c0, d = h * dk, dk
            else:
                c0, d = (nh + nkv) * dk + (h - nh - nkv) * dv, dv
            v = _f(qkv[t, c0:c0 + d]).clone()
            w = q_weight if is_q else (k_weight if is_k else None)
            if w is not None and whole:
                v = v * (inv_q if is_q else inv_k) * (w[h * dk:(h + 1) * dk] if is_q else w[(h - nh) * dk:(h - nh + 1) * dk])
            elif w is not None:
                v = v * torch.rsqrt(v.pow(2).mean() + eps) * w
            if (is_q or is_k) and cos is not None:
                half = rot // 2
                r = v.clone()
                for i in range(half):
                    a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
                    r[a] = v[a] * cos[t, i] - v[b] * sin[t, i]
                    r[b] = v[b] * cos[t, i] + v[a] * sin[t, i]
                v = r
            if is_q:
                qkv[t, c0:c0 + d] = (v * q_mult).to(qkv.dtype)
            elif cache_layer is not None:
                slot = int(slot_mapping[t])
                pg, off = slot // page_size, slot % page_size
                if is_k:
                    e0 = ((h - nh) * page_size + off) * dk
                else:
                    e0 = nkv * page_size * dk + ((h - nh - nkv) * page_size + off) * dv
                cache_layer[pg, e0:e0 + d] = v.to(cache_layer.dtype)


def masked_attention_splits(num_seqs, max_q, max_k, nh, nkv):
    return 1


def masked_attention(q, q_row_stride, cache_layer, page_size, block_table, cu_q, seqlens_k, n, num_seqs, max_q, max_k,
                     nh, nkv, dk, dv, scale, *, window=0, chunk=0, sinks=None, gate=None, splits=None, status=None, keep=0,
                     shared_kv=False):
    """shared_kv: a page holds key rows alone and a key's value is the first dv elements of its row."""
    rep = nh // nkv
    out = torch.zeros((n, nh * dv), dtype=torch.float32)
    kpart = nkv * page_size * dk
    for s in range(num_seqs):
        q0, q1, klen = int(cu_q[s]), int(cu_q[s + 1]), int(seqlens_k[s])
        qlen = q1 - q0
        for j in range(qlen):
            p = klen - qlen + j
            seen = [i for i in range(p + 1) if (window <= 0 or i > p - window or i < keep)
                    and (chunk <= 0 or i >= (p // chunk) * chunk)]
            for h in range(nh):
                g = h // rep
                qv = _f(q[q0 + j, h * dk:(h + 1) * dk])
                ks, vs = [], []
                for i in seen:
                    pg, off = int(block_table[s, i // page_size]), i % page_size
                    ks.append(_f(cache_layer[pg, (g * page_size + off) * dk:(g * page_size + off + 1) * dk]))
                    if shared_kv:
                        vs.append(ks[-1][:dv])
                    else:
                        vs.append(_f(cache_layer[pg, kpart + (g * page_size + off) * dv:kpart + (g * page_size + off + 1) * dv]))
                sc = torch.stack(ks) @ qv * scale
                mx = sc.max()
                if sinks is not None:
                    mx = torch.maximum(mx, sinks[h])
                e = torch.exp(sc - mx)
                den = e.sum() + (torch.exp(sinks[h] - mx) if sinks is not None else 0.0)
                o = (e / den) @ torch.stack(vs)
                if gate is not None:
                    o = o * torch.sigmoid(_f(gate[q0 + j, h]))
                out[q0 + j, h * dv:(h + 1) * dv] = o
    return out.to(q.dtype)


def causal_conv_silu(x, taps, bias, state, state_slots, tok_seq, cu_q, positions, max_q, status=None):
    return causal_conv(x, taps, bias, state, state_slots, tok_seq, cu_q, positions, max_q, status, act="silu")


def causal_conv(x, taps, bias, state, state_slots, tok_seq, cu_q, positions, max_q, status=None, act="none"):
    n, C = x.shape
    L = taps.shape[0]
    out = torch.zeros((n, C), dtype=torch.float32)
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        p0, slot = int(positions[r0]), int(state_slots[s])
        hist = []
        for j in range(L - 1):
            pos = p0 - (L - 1) + j
            hist.append(state[slot, j * C:(j + 1) * C].clone() if pos >= 0 else torch.zeros(C))
        for r in range(r0, r1):
            hist.append(_f(x[r]))
            acc = torch.zeros(C) if bias is None else bias.clone()
            for k in range(L):
                acc = acc + taps[k] * hist[len(hist) - L + k]
            out[r] = acc / (1.0 + torch.exp(-acc)) if act == "silu" else acc
            hist = hist[-(L - 1):] if L > 1 else []
        for j in range(L - 1):
            state[slot, j * C:(j + 1) * C] = hist[j]
    return out.to(x.dtype)


def _softplus(z):
    return torch.where(z > 20.0, z, torch.log1p(torch.exp(torch.clamp(z, max=20.0))))


def gated_delta(qkv, ab, A_log, dt_bias, state, state_offset, state_slots, cu_q, positions, nh, nkv, dk, dv,
                norm_eps=1e-6, status=None, max_q=1):
    n = qkv.shape[0]
    out = torch.zeros((n, nh * dv), dtype=torch.float32)
    rep = nh // nkv
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        slot = int(state_slots[s])
        S = state[slot, state_offset:state_offset + nh * dk * dv].view(nh, dk, dv).clone()
        if int(positions[r0]) == 0:
            S.zero_()
        for r in range(r0, r1):
            row = _f(qkv[r])
            for h in range(nh):
                g = h // rep
                qv = row[g * dk:(g + 1) * dk]
                kv = row[nkv * dk + g * dk:nkv * dk + (g + 1) * dk]
                vv = row[2 * nkv * dk + h * dv:2 * nkv * dk + (h + 1) * dv]
                qv = qv * torch.rsqrt(qv.pow(2).sum() + norm_eps) * dk ** -0.5
                kv = kv * torch.rsqrt(kv.pow(2).sum() + norm_eps)
                beta = torch.sigmoid(_f(ab[r, nh + h]))
                dec = torch.exp(-torch.exp(A_log[h]) * _softplus(_f(ab[r, h]) + dt_bias[h]))
                S[h] = dec * S[h]
                u = beta * (vv - S[h].t() @ kv)
                S[h] = S[h] + torch.outer(kv, u)
                out[r, h * dv:(h + 1) * dv] = S[h].t() @ qv
        state[slot, state_offset:state_offset + nh * dk * dv] = S.reshape(-1)
    return out


def state_space(xbc, dt, A_log, dt_bias, D, state, state_offset, state_slots, cu_q, positions, nh, groups, n_state, head,
                status=None, max_q=1):
    n = xbc.shape[0]
    out = torch.zeros((n, nh * head), dtype=torch.float32)
    rep = nh // groups
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        slot = int(state_slots[s])
        S = state[slot, state_offset:state_offset + nh * n_state * head].view(nh, n_state, head).clone()
        if int(positions[r0]) == 0:
            S.zero_()
        for r in range(r0, r1):
            row = _f(xbc[r])
            for h in range(nh):
                g = h // rep
                xv = row[h * head:(h + 1) * head]
                Bv = row[nh * head + g * n_state:nh * head + (g + 1) * n_state]
                Cv = row[nh * head + groups * n_state + g * n_state:nh * head + groups * n_state + (g + 1) * n_state]
                step = _softplus(_f(dt[r, h]) + dt_bias[h])
                S[h] = torch.exp(-torch.exp(A_log[h]) * step) * S[h] + step * torch.outer(Bv, xv)
                out[r, h * head:(h + 1) * head] = S[h].t() @ Cv + D[h] * xv
        state[slot, state_offset:state_offset + nh * n_state * head] = S.reshape(-1)
    return out


def embed_sinusoid(table, tokens, positions, freq, streams=1, status=None, pos_table=None):
    x = _f(table[tokens.long()])
    if pos_table is not None:
        x = x + _f(pos_table[positions.long()])
    if freq is not None:
        ang = positions.to(torch.float32)[:, None] * freq[None, :]
        pe = torch.stack([torch.sin(ang), torch.cos(ang)], -1).reshape(x.shape[0], -1)[:, :x.shape[1]]
        x = x + pe
    return x[:, None, :].repeat(1, streams, 1).contiguous()


def hyper_read_norm(x, y, mix, write, read, weight, eps, out_dtype, rows=None, kind="layer", branch=None):
    """x [n, S, H]: the pending write (x_t <- sum_s mix[s, t] x_s + write[t] y), then the norm of sum_s read[s] x_s.
    branch = (y2, w_y, w_y2, eps, scale): y stands for scale * (rms(y) w_y + rms(y2) w_y2)."""
    n, S, H = x.shape
    new = x
    if branch is not None:
        y2, wy, wy2, eps_y, scale = branch
        y = branch_rmsnorm_mean([y] + ([y2] if y2 is not None else []), [wy] + ([wy2] if y2 is not None else []), eps_y, scale)
    if y is not None:
        new = torch.einsum("st,nsh->nth", mix.reshape(S, S), x) + write.reshape(1, S, 1) * _f(y)[:, None, :]
        if rows is None:
            x.copy_(new)
    if weight is None:
        return None
    src = new if rows is None else new[rows.long()]
    u = src.sum(1) if read is None else (read.reshape(1, S, 1) * src).sum(1)
    if kind == "layer":
        d = u - u.mean(-1, keepdim=True)
        out = d * torch.rsqrt((d * d).mean(-1, keepdim=True) + eps) * weight
    else:
        out = u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * weight
    return out.to(out_dtype)


def branch_rmsnorm_mean(branches, weights, eps, scale):
    acc = 0
    for a, w in zip(branches, weights):
        a = _f(a)
        acc = acc + a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps) * w
    return (acc * scale).to(branches[0].dtype)


def sigmoid_gate(y, gate):
    return (_f(y) * torch.sigmoid(_f(gate))).to(y.dtype)


def softcap(x, cap):
    x.copy_(cap * torch.tanh(x / cap))
    return x


def rglru(u, y, w_a, b_a, w_i, b_i, lam, decay_c, state, state_offset, state_slots, cu_q, positions, status=None, max_q=1):
    """(In float64: 1 - a^2 loses most of its digits in float32 when a is close to 1, and a reference should not.)"""
    n, C = u.shape
    B = w_a.shape[0]
    bs = C // B
    d = torch.float64
    out = torch.zeros((n, C), dtype=d)
    sp = _softplus(lam.to(d))
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        slot = int(state_slots[s])
        S = state[slot, state_offset:state_offset + C].to(d) if int(positions[r0]) > 0 else torch.zeros(C, dtype=d)
        for r in range(r0, r1):
            ur = u[r].to(d)
            ga = torch.cat([w_a[b].to(d) @ ur[b * bs:(b + 1) * bs] for b in range(B)]) + b_a.to(d)
            gi = torch.cat([w_i[b].to(d) @ ur[b * bs:(b + 1) * bs] for b in range(B)]) + b_i.to(d)
            log_a = -decay_c * torch.sigmoid(ga) * sp
            a = torch.exp(log_a)
            S = a * S + torch.sqrt(torch.clamp(1.0 - a * a, min=0.0)) * torch.sigmoid(gi) * ur
            yr = y[r].to(d)
            out[r] = S * (0.5 * yr * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (yr + 0.044715 * yr ** 3))))
        state[slot, state_offset:state_offset + C] = S.to(state.dtype)
    return out.to(u.dtype)


def relu_squared(x):
    return (torch.relu(_f(x)) ** 2).to(x.dtype)


def moe_route(h, router, correction, experts, top, groups, keep, bias=None, score="softmax"):
    n = h.shape[0]
    if score == "chosen":
        ids = torch.zeros((n, top), dtype=torch.int32)
        wts = torch.zeros((n, top), dtype=torch.float32)
        for t in range(n):
            z = router @ _f(h[t]) + (bias if bias is not None else 0.0)
            order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
            ids[t] = torch.tensor(order, dtype=torch.int32)
            wts[t] = torch.softmax(z[order], 0)
        return ids, wts, None
    outputs = router.shape[0]
    ids = torch.zeros((n, top), dtype=torch.int32)
    wts = torch.zeros((n, top), dtype=torch.float32)
    per = outputs // groups
    for t in range(n):
        s = torch.softmax(router @ _f(h[t]) + (bias if bias is not None else 0.0), 0)
        choice = s + (correction if correction is not None else 0.0)
        if groups > 1 and keep < groups:
            gs = choice.reshape(groups, per).max(1).values
            kept = sorted(range(groups), key=lambda g: (-float(gs[g]), g))[:keep]
            for g in range(groups):
                if g not in kept:
                    choice[g * per:(g + 1) * per] = -math.inf
        order = sorted(range(outputs), key=lambda e: (-float(choice[e]), e))[:top]
        ids[t] = torch.tensor(order, dtype=torch.int32)
        wts[t] = s[order] / (s[order].sum() + 1e-20)
    return ids, wts, None


def moe_table_route(tokens, table, experts, status=None):
    """ids = table[token], each with weight 1 / top; no plan is needed by the restatement of the experts."""
    ids = table[tokens.long()].to(torch.int32)
    return ids, torch.full(ids.shape, 1.0 / ids.shape[1], dtype=torch.float32), None


def moe_experts(h, ids, wts, plan, w_up, w_down, shared=None, gated=False, act=(0.0, 1.0, 0.0)):
    """act = (limit, alpha, shift): a gated expert's hidden row is g' * sigmoid(alpha g') * (u' + shift) with g' = min(g, limit)
    and u' = clamp(u, -limit, limit) when limit > 0."""
    limit, alpha, shift = act
    n, W = h.shape
    experts = 0 if w_up is None else w_up.shape[0]
    out = torch.zeros((n, W), dtype=torch.float32)
    for t in range(n):
        for e, g in zip(ids[t].tolist(), wts[t].tolist()):
            if e >= experts:
                out[t] += g * _f(h[t])
            elif gated:
                gu = _f(w_up[e]) @ _f(h[t])
                gg, uu = gu[0::2], gu[1::2]
                if limit > 0:
                    gg, uu = torch.clamp(gg, max=limit), torch.clamp(uu, min=-limit, max=limit)
                hid = (gg / (1.0 + torch.exp(-alpha * gg)) * (uu + shift)).to(h.dtype)
                out[t] += g * (_f(w_down[e]) @ _f(hid))
            else:
                hid = (torch.relu(_f(w_up[e]) @ _f(h[t])) ** 2).to(h.dtype)
                out[t] += g * (_f(w_down[e]) @ _f(hid))
    if shared is not None:
        out += _f(shared)
    return out.to(h.dtype)


def _logsigmoid(z):
    return torch.clamp(z, max=0.0) - torch.log1p(torch.exp(-z.abs()))


def matrix_memory(qkv, gates, gate_bias, cap, state, state_slots, cu_q, positions, nh, dk, dv, q_scale, floor_eps=1e-6,
                  status=None, max_q=1):
    n = qkv.shape[0]
    out = torch.zeros((n, nh * dv), dtype=torch.float32)
    nS, nn = nh * dk * dv, nh * dk
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        slot = int(state_slots[s])
        S = state[slot, :nS].view(nh, dv, dk).transpose(1, 2).clone()          # the slot holds S column by column
        nv = state[slot, nS:nS + nn].view(nh, dk).clone()
        m = state[slot, nS + nn:nS + nn + nh].clone()
        if int(positions[r0]) == 0:
            S.zero_(); nv.zero_(); m.zero_()
        for r in range(r0, r1):
            row = _f(qkv[r])
            a = gates[r] + (gate_bias if gate_bias is not None else 0.0)
            for h in range(nh):
                qv = row[h * dk:(h + 1) * dk] * q_scale
                kv = row[nh * dk + h * dk:nh * dk + (h + 1) * dk]
                vv = row[2 * nh * dk + h * dv:2 * nh * dk + (h + 1) * dv]
                li = cap * torch.tanh(a[h] / cap)
                lf = _logsigmoid(cap * torch.tanh(a[nh + h] / cap))
                new = torch.maximum(lf + m[h], li)
                keep, take = torch.exp(lf + m[h] - new), torch.exp(li - new)
                S[h] = keep * S[h] + take * torch.outer(kv, vv)
                nv[h] = keep * nv[h] + take * kv
                m[h] = new
                den = torch.maximum((nv[h] @ qv).abs(), torch.exp(-new)) + floor_eps
                out[r, h * dv:(h + 1) * dv] = (S[h].t() @ qv) / den
        state[slot, :nS] = S.transpose(1, 2).reshape(-1)
        state[slot, nS:nS + nn] = nv.reshape(-1)
        state[slot, nS + nn:nS + nn + nh] = m
    return out


def gated_linear_attention(qkv, decay_logits, tau, state, state_slots, cu_q, positions, nh, dk, dv, q_scale, status=None,
                           max_q=1):
    n = qkv.shape[0]
    out = torch.zeros((n, nh * dv), dtype=torch.float32)
    nS = nh * dk * dv
    for s in range(cu_q.numel() - 1):
        r0, r1 = int(cu_q[s]), int(cu_q[s + 1])
        if r1 == r0:
            continue
        slot = int(state_slots[s])
        S = state[slot, :nS].view(nh, dv, dk).transpose(1, 2).clone()          # the slot holds S column by column
        if int(positions[r0]) == 0:
            S.zero_()
        for r in range(r0, r1):
            row = _f(qkv[r])
            alpha = torch.exp(_logsigmoid(decay_logits[r]) / tau).view(nh, dk)
            for h in range(nh):
                qv = row[h * dk:(h + 1) * dk] * q_scale
                kv = row[nh * dk + h * dk:nh * dk + (h + 1) * dk]
                vv = row[2 * nh * dk + h * dv:2 * nh * dk + (h + 1) * dv]
                S[h] = alpha[h][:, None] * S[h] + torch.outer(kv, vv)
                out[r, h * dv:(h + 1) * dv] = S[h].t() @ qv
        state[slot, :nS] = S.transpose(1, 2).reshape(-1)
    return out


ALL = ["matrix_memory", "gated_linear_attention", "embed", "resolve_tokens", "sample_truncated", "add_rmsnorm", "add_residual", "add_residual_ss", "skinny_applies", "tc_applies", "few_rows_applies", "swiglu", "linear", "strict_fp32", "rope_cos_sin",
       "qk_norm_rope_write", "attention_splits", "paged_attention", "shortconv", "sample_rows",
       "apply_penalties", "postnorm_add_rmsnorm", "gated_group_rmsnorm", "scale_rows", "rope_cos_sin_scaled",
       "qk_norm_rope_write_split", "masked_attention_splits", "masked_attention", "causal_conv_silu", "gated_delta",
       "state_space", "causal_conv", "embed_sinusoid", "hyper_read_norm", "branch_rmsnorm_mean", "sigmoid_gate", "softcap",
       "rglru", "relu_squared", "moe_route", "moe_experts", "moe_table_route", "scaled_add_rmsnorm", "latent_prepare",
       "latent_rotate_q", "head_products", "latent_attention"]
