"""Plain PyTorch float32 statements of the package's operations, with the same
signatures as `sllm_b200.ops`.

Two uses, both in tests only: (1) the reference each CUDA kernel is compared
with, on the GPU, at sizes other than the engine's; (2) patched over
`sllm_b200.ops` (fixture `cpu_ops`), they let the step function, the cache and
the scheduler be exercised on a machine without a GPU.  The product never
imports this file; without its kernels it raises.
"""

from __future__ import annotations

import torch


def embed_gather(table, ids, scale=1.0):
    return table[ids.long()].float() * scale


def add_sinusoid_(stream, positions, inv_freq):
    ang = positions.float()[:, None] * inv_freq[None, :]
    stream[:, 0::2] += torch.sin(ang)
    stream[:, 1::2] += torch.cos(ang)
    return stream


def add_group_ssq(stream, terms, groups, eps, want_rinv=True):
    for t in (terms or ()):
        if t is not None:
            stream += t.float().sum(0) if t.dim() == 3 else t.float()
    if not want_rinv:
        return None
    T, W = stream.shape
    return (stream.reshape(T, groups, W // groups).pow(2).mean(-1) + eps).rsqrt()


def group_norm_shift(stream, rinv, gain, out_dtype, *, groups=None, eps=0.0, mix=None, state=None, step=None, want_plain=True):
    T, W = stream.shape
    if rinv is None:
        rinv = (stream.reshape(T, groups, W // groups).pow(2).mean(-1) + eps).rsqrt()
    groups = rinv.shape[1]
    h = (stream.reshape(T, groups, W // groups) * rinv[:, :, None]).reshape(T, W) * gain
    if mix is None:
        return h.to(out_dtype)
    prev = torch.empty_like(h)
    prev[1:] = h[:-1]
    starts = step.q_start.long().tolist()
    for s in range(step.num_seqs):
        slot = int(step.state_slots[s])
        prev[starts[s]] = state[slot]
        state[slot] = h[starts[s + 1] - 1]
    hs = h + (prev - h) * mix
    return (h.to(out_dtype) if want_plain else None), hs.to(out_dtype)


def act_mul(gu, interleave, out_dtype, act):
    T, two_i = gu.shape
    I = two_i // 2
    v = gu.float().reshape(T, I // interleave, 2, interleave)
    g, u = v[:, :, 0, :], v[:, :, 1, :]
    if act == "silu":
        a = g / (1.0 + torch.exp(-g))
    else:
        a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    return (a * u).reshape(T, I).to(out_dtype)


def linear_act_mul(x, w_gate_up, bias, interleave, out_dtype, act):
    return act_mul(linear(x, w_gate_up, bias, x.dtype), interleave, out_dtype, act)


def tanh_cols(x, col0, n, out_dtype):
    return torch.tanh(x[:, col0:col0 + n]).to(out_dtype)


def delta_rule(proj, offs, decay, a_bias, state, step, heads, dk, dv):
    T = proj.shape[0]
    off_r, off_k, off_v, off_a = offs
    C = heads * dk
    r = proj[:, off_r:off_r + C].reshape(T, heads, dk)
    k = proj[:, off_k:off_k + C].reshape(T, heads, dk)
    v = proj[:, off_v:off_v + heads * dv].reshape(T, heads, dv)
    a = torch.sigmoid(proj[:, off_a:off_a + C] + a_bias).reshape(T, heads, dk)
    d = torch.exp(-float(torch.exp(torch.tensor(-0.5))) * torch.sigmoid(decay)).reshape(T, heads, dk)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    out = torch.empty((T, heads, dv), dtype=torch.float32, device=proj.device)
    starts = step.q_start.long().tolist()
    for s in range(step.num_seqs):
        slot = int(step.state_slots[s])
        S = state[slot].clone()
        for t in range(starts[s], starts[s + 1]):
            uS = torch.einsum("hi,hij->hj", u[t], S)
            S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hij,hi->hj", S, r[t])
        state[slot] = S
    return out.reshape(T, heads * dv)


def delta_out(o, gain, proj, off_g, eps, heads, dv, out_dtype, gate_act="sigmoid", out=None, out_off=0):
    T = o.shape[0]
    x = o.reshape(T, heads, dv)
    x = x * (x.pow(2).mean(-1, keepdim=True) + eps).rsqrt()
    if gate_act == "none":
        gate = 1.0
    else:
        g = proj[:, off_g:off_g + heads * dv]
        gate = torch.sigmoid(g) if gate_act == "sigmoid" else g * torch.sigmoid(g)
    y = x.reshape(T, heads * dv) * gain * gate
    if out is None:
        return y.to(out_dtype)
    out[:, out_off:out_off + heads * dv] = y.to(out.dtype)
    return out


def forget_gate_attention(proj, offs, f_bias, lower, state, step, heads, dk, dv):
    T = proj.shape[0]
    off_q, off_f, off_v = offs
    q = proj[:, off_q:off_q + heads * dk]
    q = (q * torch.sigmoid(q)).reshape(T, heads, dk)
    f = (lower + (1.0 - lower) * torch.sigmoid(proj[:, off_f:off_f + heads * dk] + f_bias)).reshape(T, heads, dk)
    v = proj[:, off_v:off_v + heads * dv].reshape(T, heads, dv)
    out = torch.empty((T, heads, dv), dtype=torch.float32, device=proj.device)

    def token(t, S):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        return S, torch.einsum("hij,hi->hj", S, q[t])
    _walk(step, state, out, token)
    return out.reshape(T, heads * dv)


def add_rows_(stream, rows, vec):
    if rows is not None:
        stream += rows
    if vec is not None:
        stream += vec


def norm_pair(stream, gain_a, gain_b, eps, out_dtype):
    x = stream * (stream.pow(2).mean(-1, keepdim=True) + eps).rsqrt()
    return (x * gain_a).to(out_dtype), ((x * gain_b).to(out_dtype) if gain_b is not None else None)


def _walk(step, state, out, token):
    """Request by request, token by token: ``token(t, S) -> (S, o)`` from and into the requests' state rows."""
    starts = step.q_start.long().tolist()
    for s in range(step.num_seqs):
        slot = int(step.state_slots[s])
        S = state[slot].clone()
        for t in range(starts[s], starts[s + 1]):
            S, out[t] = token(t, S)
        state[slot] = S


def gated_delta_rule(qkv, offs, gates, off_b, off_dt, a_log, dt_bias, state, step, heads, key_heads, dk, dv, q_scale):
    T = qkv.shape[0]
    off_q, off_k, off_v = offs
    rep = heads // key_heads
    q = qkv[:, off_q:off_q + key_heads * dk].reshape(T, key_heads, dk)
    k = qkv[:, off_k:off_k + key_heads * dk].reshape(T, key_heads, dk)
    v = qkv[:, off_v:off_v + heads * dv].reshape(T, heads, dv)
    q = (q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * q_scale).repeat_interleave(rep, dim=1)
    k = (k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(gates[:, off_b:off_b + heads])
    g = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(gates[:, off_dt:off_dt + heads] + dt_bias))
    out = torch.empty((T, heads, dv), dtype=torch.float32, device=qkv.device)

    def token(t, S):
        S = g[t][:, None, None] * S
        w = beta[t][:, None] * (v[t] - torch.einsum("hij,hi->hj", S, k[t]))
        S = S + k[t][:, :, None] * w[:, None, :]
        return S, torch.einsum("hij,hi->hj", S, q[t])
    _walk(step, state, out, token)
    return out.reshape(T, heads * dv)


def gated_linear_attention(proj, offs, z, state, step, heads, dk, dv, q_scale, tau):
    T = proj.shape[0]
    off_q, off_k, off_v = offs
    q = proj[:, off_q:off_q + heads * dk].reshape(T, heads, dk) * q_scale
    k = proj[:, off_k:off_k + heads * dk].reshape(T, heads, dk)
    v = proj[:, off_v:off_v + heads * dv].reshape(T, heads, dv)
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).reshape(T, heads, dk)
    out = torch.empty((T, heads, dv), dtype=torch.float32, device=proj.device)

    def token(t, S):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        return S, torch.einsum("hij,hi->hj", S, q[t])
    _walk(step, state, out, token)
    return out.reshape(T, heads * dv)


def qk_norm_rope_kv_write(qkv, q_gain, k_gain, eps, positions, table, rotary_dim, nq, nkv, dim, vdim, slot_mapping, k_cache, v_cache,
                          out_dtype, q_mul=None, col_off=0):
    qkv = qkv[:, col_off:]
    T = qkv.shape[0]
    D = k_cache.shape[3]
    qk = qkv[:, :(nq + nkv) * dim].float().reshape(T, nq + nkv, dim)
    v = qkv[:, (nq + nkv) * dim:(nq + nkv) * dim + nkv * vdim].float().reshape(T, nkv, vdim)
    if q_gain is not None:
        qk = qk * (qk.pow(2).mean(-1, keepdim=True) + eps).rsqrt()
        qk = torch.cat([qk[:, :nq] * q_gain, qk[:, nq:] * k_gain], dim=1)
    if q_mul is not None:
        qk = torch.cat([qk[:, :nq] * q_mul[None, :, None], qk[:, nq:]], dim=1)
    if rotary_dim:
        half = rotary_dim // 2
        cs = table[positions.long()]
        c, s = cs[:, None, 0, :], cs[:, None, 1, :]
        x1, x2 = qk[..., :half], qk[..., half:rotary_dim]
        qk = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, qk[..., rotary_dim:]], dim=-1)
    qk = torch.nn.functional.pad(qk, (0, D - dim))
    v = torch.nn.functional.pad(v, (0, D - vdim))
    if slot_mapping is not None:
        ps = k_cache.shape[2]
        ok = slot_mapping >= 0
        page, off = slot_mapping[ok].long() // ps, slot_mapping[ok].long() % ps
        k_cache[page, :, off, :] = qk[ok][:, nq:].to(k_cache.dtype)
        v_cache[page, :, off, :] = v[ok].to(v_cache.dtype)
    return qk[:, :nq].reshape(T, nq * D).to(out_dtype)


def short_conv_silu(x, off, weight, state, step):
    C, taps = weight.shape
    T = x.shape[0]
    out = torch.empty((T, C), dtype=torch.float32, device=x.device)
    starts = step.q_start.long().tolist()
    for s in range(step.num_seqs):
        a, b = starts[s], starts[s + 1]
        slot = int(step.state_slots[s])
        xs = x[a:b, off:off + C].float()
        before = state[slot].t() if taps > 1 else xs[:0]                 # [taps-1, C], oldest first
        padded = torch.cat([before, xs], dim=0)
        acc = torch.zeros((b - a, C), dtype=torch.float32, device=x.device)
        for j in range(taps):
            acc += padded[j:j + b - a] * weight[:, j]
        out[a:b] = acc * torch.sigmoid(acc)
        if taps > 1:
            state[slot] = padded[padded.shape[0] - (taps - 1):].t()
    return out


def norm_mean_add_(stream, a, gain_a, b, gain_b, eps):
    na = a * (a.pow(2).mean(-1, keepdim=True) + eps).rsqrt() * gain_a
    nb = b * (b.pow(2).mean(-1, keepdim=True) + eps).rsqrt() * gain_b
    stream += 0.5 * (na + nb)


def moe_route(logits, correction, groups, keep, top, scale):
    T, E = logits.shape
    s = torch.sigmoid(logits.float())
    choice = s + correction
    if groups > 1 and keep < groups:
        per = E // groups
        grouped = choice.reshape(T, groups, per)
        score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros((T, groups), dtype=torch.bool, device=logits.device)
        allowed.scatter_(1, best, True)
        choice = torch.where(allowed.repeat_interleave(per, dim=1), choice, torch.full_like(choice, float("-inf")))
    idx = torch.sort(-choice, dim=-1, stable=True).indices[:, :top]
    wts = s.gather(1, idx) * scale
    dense = torch.zeros((T, E), dtype=torch.float32, device=logits.device)
    dense.scatter_(1, idx, wts)
    return dense, idx.int(), wts


def moe_act(up, dense, ff, out_dtype):
    T, N = up.shape
    E = dense.shape[1]
    w = torch.ones((T, N), dtype=torch.float32, device=up.device)
    w[:, :E * ff] = dense.repeat_interleave(ff, dim=1)
    return (torch.nn.functional.gelu(up.float()) * w).to(out_dtype)


def latent_write(proj, off, rank, gain, eps, slot_mapping, cache):
    x = proj[:, off:off + rank]
    c = x * (x.pow(2).mean(-1, keepdim=True) + eps).rsqrt() * gain
    ps = cache.shape[2]
    ok = slot_mapping >= 0
    slots = slot_mapping[ok].long()
    cache[slots // ps, 0, slots % ps, :] = c[ok].to(cache.dtype)


def head_linear(x, xoff, w, out_dtype, *, gate=None, goff=0, gate_elem=False, xstride=None, ostride=None):
    H, dout, din = w.shape
    T = x.shape[0]
    xs_, os_ = xstride or din, ostride or dout
    xs = x[:, xoff:xoff + H * xs_].reshape(T, H, xs_)[:, :, :din].to(w.dtype).float()      # (operands in the matrix's dtype)
    out = torch.einsum("thi,hoi->tho", xs, w.float())
    if gate is not None and gate_elem:
        out = out * torch.sigmoid(gate[:, goff:goff + H * dout]).reshape(T, H, dout)
    elif gate is not None:
        out = out * torch.sigmoid(gate[:, goff:goff + H])[:, :, None]
    full = torch.zeros((T, H, os_), dtype=out_dtype, device=x.device)
    full[:, :, :dout] = out.to(out_dtype)
    return full.reshape(T, H * os_)


def _rotate(x, positions, table, rot):
    """x [..., n]: the first ``rot`` channels in the rotate-half layout by ``table`` [positions, 2, rot/2]."""
    if not rot:
        return x
    half = rot // 2
    cs = table[positions.long()]                       # [T, 2, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, sn = cs[:, 0].reshape(shape), cs[:, 1].reshape(shape)
    u, v = x[..., :half], x[..., half:rot]
    return torch.cat([u * c - v * sn, v * c + u * sn, x[..., rot:]], dim=-1)


def latent_rope_write(proj, off, rank, tail, rotary_dim, gain, eps, positions, table, slot_mapping, cache):
    x = proj[:, off:off + rank]
    c = x * (x.pow(2).mean(-1, keepdim=True) + eps).rsqrt() * gain
    row = torch.zeros((proj.shape[0], cache.shape[3]), dtype=torch.float32, device=proj.device)
    row[:, :rank] = c
    row[:, rank:rank + tail] = _rotate(proj[:, off + rank:off + rank + tail].float(), positions, table, rotary_dim)
    ps = cache.shape[2]
    ok = slot_mapping >= 0
    slots = slot_mapping[ok].long()
    cache[slots // ps, 0, slots % ps, :] = row[ok].to(cache.dtype)


def rope_cols_(out, ooff, ostride, x, xoff, xstride, n, rotary_dim, positions, table, heads):
    T = x.shape[0]
    src = x[:, xoff:].float()
    o = out.reshape(T, heads, ostride)
    for h in range(heads):
        o[:, h, ooff:ooff + n] = _rotate(src[:, h * xstride:h * xstride + n], positions, table, rotary_dim).to(out.dtype)
        o[:, h, ooff + n:] = 0


def short_conv_add(x, weight, state, step, out_dtype):
    C, taps = weight.shape
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    starts = step.q_start.long().tolist()
    for s in range(step.num_seqs):
        a, b = starts[s], starts[s + 1]
        slot = int(step.state_slots[s])
        xs = x[a:b].float()
        before = state[slot].t() if taps > 1 else xs[:0]                 # [taps-1, C], oldest first
        padded = torch.cat([before, xs], dim=0)
        acc = xs.clone()
        for j in range(taps):
            acc += padded[j:j + b - a] * weight[:, j]
        out[a:b] = acc
        if taps > 1:
            state[slot] = padded[padded.shape[0] - (taps - 1):].t()
    return out.to(out_dtype)


def moe_route_top_softmax(logits, top, scale=1.0):
    T, E = logits.shape
    idx = torch.sort(-logits.float(), dim=-1, stable=True).indices[:, :top]
    wts = torch.softmax(logits.float().gather(1, idx), dim=-1) * scale
    dense = torch.zeros((T, E), dtype=torch.float32, device=logits.device)
    dense.scatter_(1, idx, wts)
    return dense, idx.int(), wts


def gated_clamp_act(gu, interleave, limit, out_dtype, *, alpha=1.702, dense=None, ff=None, act="clamped_swish"):
    T, two_n = gu.shape
    N = two_n // 2
    v = gu.float().reshape(T, N // interleave, 2, interleave)
    if act == "silu":
        g, u = v[:, :, 0, :].reshape(T, N), v[:, :, 1, :].reshape(T, N)
        y = g * torch.sigmoid(g) * u
    else:
        g = v[:, :, 0, :].reshape(T, N).clamp(max=limit)
        u = v[:, :, 1, :].reshape(T, N).clamp(-limit, limit)
        y = g * torch.sigmoid(alpha * g) * (u + 1.0)
    if dense is not None:
        y = y * dense.repeat_interleave(ff, dim=1)
    return y.to(out_dtype)


def post_add_norm(stream, term, post_gain, post_eps, pre_gain, pre_eps, out_dtype=torch.float32):
    if term is not None:
        t = term.float().sum(0) if term.dim() == 3 else term.float()
        stream += t * (t.pow(2).mean(-1, keepdim=True) + post_eps).rsqrt() * post_gain
    if pre_gain is None:
        return None
    return (stream * (stream.pow(2).mean(-1, keepdim=True) + pre_eps).rsqrt() * pre_gain).to(out_dtype)


def post_add_norm_conv(stream, term, post_gain, post_eps, pre_gain, pre_eps, weight, state, step, out_dtype):
    assert stream.shape[0] == step.num_seqs, "one token a request"
    h = post_add_norm(stream, term, post_gain, post_eps, pre_gain, pre_eps, torch.float32)
    return short_conv_add(h, weight, state, step, out_dtype)


def mingru_scan(proj, offs, state, step, width, out_dtype):
    oz, ox, og = offs
    z = torch.sigmoid(proj[:, oz:oz + width])
    b = proj[:, ox:ox + width]
    cand = torch.where(b >= 0, b + 0.5, torch.sigmoid(b))
    g = proj[:, og:og + width]
    out = torch.empty((proj.shape[0], width), dtype=torch.float32, device=proj.device)

    def token(t, S):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        return S, S * g[t] * torch.sigmoid(g[t])
    _walk(step, state, out, token)
    return out.to(out_dtype)


def decay_linear_attention(proj, offs, decay, state, step, heads, dk, dv):
    T = proj.shape[0]
    off_q, off_k, off_v = offs
    act = torch.nn.functional.silu
    q = act(proj[:, off_q:off_q + heads * dk]).reshape(T, heads, dk)
    k = act(proj[:, off_k:off_k + heads * dk]).reshape(T, heads, dk)
    v = act(proj[:, off_v:off_v + heads * dv]).reshape(T, heads, dv)
    out = torch.empty((T, heads, dv), dtype=torch.float32, device=proj.device)

    def token(t, S):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        return S, torch.einsum("hij,hi->hj", S, q[t])
    _walk(step, state, out, token)
    return out.reshape(T, heads * dv)


def add_rmsnorm(residual, delta, weight, eps, out_dtype):
    if delta is not None:
        d = delta.float()
        if d.dim() == 3:
            d = d.sum(0)
        residual += d
    var = (residual * residual).mean(-1, keepdim=True)
    return (residual * (var + eps) ** -0.5 * weight).to(out_dtype)


def linear(x, w, bias, out_dtype, allow_partials=False):
    out = x.float() @ w.float().t()
    if bias is not None:
        out = out + bias
    return out.to(out_dtype)


def can_accumulate(x, w):
    return x.dtype == torch.bfloat16 and x.shape[0] <= 8 and x.shape[1] % 32 == 0 and 16 <= w.shape[0] <= 8192


def linear_accumulate(x, w, bias, residual):
    residual += linear(x, w, bias, torch.float32)


def silu_mul(gu, interleave, out_dtype):
    T, two_i = gu.shape
    I = two_i // 2
    v = gu.float().reshape(T, I // interleave, 2, interleave)
    g, u = v[:, :, 0, :], v[:, :, 1, :]
    return (g * (1.0 / (1.0 + torch.exp(-g))) * u).reshape(T, I).to(out_dtype)


def linear_silu_mul(x, w_gate_up, interleave, out_dtype):
    return silu_mul(linear(x, w_gate_up, None, x.dtype), interleave, out_dtype)


def rope_kv_write(qkv, bias, positions, table, rotary_dim, nq, nkv, hd, slot_mapping, k_cache, v_cache, out_dtype):
    x = qkv.float()
    if x.dim() == 3:
        x = x.sum(0)
    T = x.shape[0]
    if bias is not None:
        x = x + bias
    x = x.reshape(T, nq + 2 * nkv, hd)
    if rotary_dim:
        half = rotary_dim // 2
        cs = table[positions.long()]                     # [T, 2, half]
        c, s = cs[:, None, 0, :], cs[:, None, 1, :]
        qk = x[:, :nq + nkv]
        x1, x2 = qk[..., :half], qk[..., half:rotary_dim]
        rot = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, qk[..., rotary_dim:]], dim=-1)
        x = torch.cat([rot, x[:, nq + nkv:]], dim=1)
    q = x[:, :nq].reshape(T, nq * hd).to(out_dtype)
    if slot_mapping is not None:
        ps = k_cache.shape[2]
        page, off = slot_mapping.long() // ps, slot_mapping.long() % ps
        k_cache[page, :, off, :] = x[:, nq:nq + nkv].to(k_cache.dtype)
        v_cache[page, :, off, :] = x[:, nq + nkv:].to(v_cache.dtype)
    return q


def attention_simt(q, k_cache, v_cache, block_tables, positions, seq_of_token, nq, nkv, hd, scale, window, block=None, sink=None):
    T = q.shape[0]
    ps = k_cache.shape[2]
    out = torch.empty((T, nq, hd), dtype=torch.float32, device=q.device)
    qf = q.float().reshape(T, nq, hd)
    rep = nq // nkv
    for t in range(T):
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        if block:
            lo = max(lo, pos // block * block)
        j = torch.arange(lo, pos + 1, device=q.device)
        pages = block_tables[int(seq_of_token[t])].long()[j // ps]
        k = k_cache[pages, :, j % ps, :].float()          # [n, nkv, hd]
        v = v_cache[pages, :, j % ps, :].float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        s = torch.einsum("hd,nhd->hn", qf[t], k) * scale
        if sink is not None:                               # one more term of the denominator: no key, no value, not scaled
            p = torch.softmax(torch.cat([s, sink.float()[:, None]], dim=-1), dim=-1)[:, :-1]
        else:
            p = torch.softmax(s, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", p, v)
    return out.reshape(T, nq * hd).to(q.dtype)


def paged_attention(q, k_cache, v_cache, step, group, nq, nkv, hd, scale, window, block=None, sink=None):
    g = step.groups[group]
    return attention_simt(q, k_cache, v_cache, g.block_tables, step.positions, step.seq_of_token,
                          nq, nkv, hd, scale, window, block, sink)


def pool_kv_write(k_cache, v_cache, step, group, pk_cache, pv_cache, pool_group, pool):
    g, pg = step.groups[group], step.groups[pool_group]
    ps = k_cache.shape[2]
    for t in range(step.num_tokens):
        slot = int(pg.slot_mapping[t])
        if slot < 0:
            continue
        pos = int(step.positions[t])
        j = torch.arange(pos - pool + 1, pos + 1, device=k_cache.device)
        pages = g.block_tables[int(step.seq_of_token[t])].long()[j // ps]
        pk_cache[slot // ps, :, slot % ps, :] = k_cache[pages, :, j % ps, :].float().mean(0).to(pk_cache.dtype)
        pv_cache[slot // ps, :, slot % ps, :] = v_cache[pages, :, j % ps, :].float().mean(0).to(pv_cache.dtype)


def pooled_attention(q, k_cache, v_cache, pk_cache, pv_cache, step, group, pool_group, nq, nkv, vdim, scale, window, pool, sink=None,
                     out_scale=1.0, out=None, out_off=0):
    g = step.groups[group]
    pg = step.groups[pool_group] if (pool_group is not None and window) else None
    T = q.shape[0]
    ps, D = k_cache.shape[2], k_cache.shape[3]
    res = torch.empty((T, nq, vdim), dtype=torch.float32, device=q.device)
    qf = q.float().reshape(T, nq, D)
    rep = nq // nkv
    for t in range(T):
        pos, seq = int(step.positions[t]), int(step.seq_of_token[t])
        lo = max(0, pos - window + 1) if window else 0
        j = torch.arange(lo, pos + 1, device=q.device)
        pages = g.block_tables[seq].long()[j // ps]
        k, v = k_cache[pages, :, j % ps, :].float(), v_cache[pages, :, j % ps, :].float()
        nb = lo // pool if pg is not None else 0
        if nb:
            b = torch.arange(nb, device=q.device)
            bp = pg.block_tables[seq].long()[b // ps]
            k = torch.cat([pk_cache[bp, :, b % ps, :].float(), k], dim=0)
            v = torch.cat([pv_cache[bp, :, b % ps, :].float(), v], dim=0)
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)[..., :vdim]
        s = torch.einsum("hd,nhd->hn", qf[t], k) * scale
        if sink is not None:
            p = torch.softmax(torch.cat([s, sink.float()[:, None]], dim=-1), dim=-1)[:, :-1]
        else:
            p = torch.softmax(s, dim=-1)
        res[t] = torch.einsum("hn,nhd->hd", p, v) * out_scale
    res = res.reshape(T, nq * vdim)
    if out is None:
        return res.to(q.dtype)
    out[:, out_off:out_off + nq * vdim] = res.to(out.dtype)
    return out


def gather_rows(x, rows):
    if x.dim() == 3:
        return x[:, rows.long()].sum(0)
    return x[rows.long()].clone()


def sample_rows(logits, temperature=None, uniform=None, top_k=None, top_p=None):
    from tests.plain import qwen2_plain as plain
    R, V = logits.shape
    out = torch.empty(R, dtype=torch.int32, device=logits.device)
    for r in range(R):
        t = float(temperature[r]) if temperature is not None else 0.0
        k = int(top_k[r]) if top_k is not None and int(top_k[r]) > 0 else None
        p = float(top_p[r]) if top_p is not None and float(top_p[r]) >= 0 else None
        out[r] = plain.sample(logits[r].double().cpu().numpy(), t, k, p, u=float(uniform[r]) if t > 0 else None)
    return out


def repetition_penalty_(logits, pair_row, pair_id, pair_penalty):
    V = logits.shape[1]
    for r, i, q in zip(pair_row.tolist(), pair_id.tolist(), pair_penalty.tolist()):
        if 0 <= i < V:
            v = float(logits[r, i])
            logits[r, i] = v * q if v < 0 else v / q
    return logits


def mark_seen(seen, step):
    slots = step.state_slots[step.seq_of_token[:step.num_tokens].long()].long()
    ids = step.token_ids[:step.num_tokens].long()
    ok = (ids >= 0) & (ids < seen.shape[1]) & (slots >= 0) & (slots < seen.shape[0])
    seen[slots[ok], ids[ok]] = 1


def penalty_from_seen_(logits, seen, step, penalty):
    for r in range(logits.shape[0]):
        q = float(penalty[r])
        if not q > 0 or q == 1.0:
            continue
        slot = int(step.state_slots[step.seq_of_token[step.logit_rows[r]]])
        mine = seen[slot].bool()
        row = logits[r].double()
        logits[r] = torch.where(mine, torch.where(row < 0, row * q, row / q), row).float()
    return logits


ALL = ["forget_gate_attention", "add_rows_", "norm_pair", "pool_kv_write", "pooled_attention", "post_add_norm_conv", "latent_rope_write", "rope_cols_", "short_conv_add", "moe_route_top_softmax", "gated_clamp_act", "post_add_norm", "mingru_scan",
       "decay_linear_attention", "gated_delta_rule", "gated_linear_attention", "qk_norm_rope_kv_write", "short_conv_silu", "norm_mean_add_", "moe_route", "moe_act",
       "add_sinusoid_", "add_group_ssq", "group_norm_shift", "act_mul", "linear_act_mul", "tanh_cols", "delta_rule", "delta_out", "latent_write",
       "head_linear", "embed_gather", "add_rmsnorm", "linear", "can_accumulate", "linear_accumulate", "silu_mul", "linear_silu_mul", "rope_kv_write",
       "attention_simt", "paged_attention", "gather_rows", "sample_rows", "repetition_penalty_", "mark_seen", "penalty_from_seen_"]
