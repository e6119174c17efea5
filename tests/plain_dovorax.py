"""Dovorax, plainly: every mechanism as one slow function in float64, written from the design's equations
and sharing nothing with the engine.  W maps tensor names to torch tensors; tokens is a list of ids.

Notation: x the residual stream [T, width]; N(w, y) = w * y / sqrt(mean(y^2) + eps) over the last axis;
N1(w, y) = N(1 + w, y) (a weight stored around zero); U(y) = N(1, y).

    x = embed[token]
    per layer: x <- N1(w_1, alpha x + mixer(x));  x <- N1(w_2, alpha x + ff(x))     (the norm comes after the sum)
    logits = embed N1(w_f, x)
"""
import math

import torch

F = torch.float64


def rms_norm(y, w, eps, one_plus=False):
    y = y.to(F)
    scale = 1.0 if w is None else (w.to(F) + 1.0 if one_plus else w.to(F))
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * scale


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def logsigmoid(z):
    return -softplus(-z)


def lin(h, W, name):
    return h.to(F) @ W[name].to(F).T


def rotary(rot):
    """-> (frequencies [dims/2], magnitude): f_i = base^(-2i/dims); with ``scaling`` the frequencies between a fast
    and a slow turn count over the original length are blended towards f_i / factor along a ramp over the pair
    index, and cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F), 1.0
    index = lambda turns: dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(index(sc["fast"])), 0)
    hi = min(math.ceil(index(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, rot, first_position=0):
    """x [T, heads, d]: the first rot.dims elements of every head turned, pair i being (i, i + dims/2)."""
    x = x.to(F).clone()
    T, dims = x.shape[0], rot["dims"]
    half = dims // 2
    f, mag = rotary(rot)
    ang = (torch.arange(T, dtype=F) + first_position)[:, None] * f[None, :]
    c, s = mag * torch.cos(ang)[:, None, :], mag * torch.sin(ang)[:, None, :]
    u, v = x[..., :half].clone(), x[..., half:dims].clone()
    x[..., :half] = u * c - v * s
    x[..., half:dims] = v * c + u * s
    return x


def short_conv(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F), u.to(F)])
    y = sum(w[:, j].to(F)[None, :] * padded[j:j + T] for j in range(taps))
    return y if bias is None else y + bias.to(F)


def visible(T, window):
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    return (d >= 0) & (d < window) if window else d >= 0


def softmax_rows(s, mask, one_more=False):
    """Softmax over the visible keys; one_more: one further term exp(0) in the denominator."""
    s = s.masked_fill(~mask, -math.inf)
    top = s.max(-1, keepdim=True).values
    if one_more:
        top = torch.clamp(top, min=0.0)
    e = torch.exp(s - top)
    den = e.sum(-1, keepdim=True)
    return e / (den + torch.exp(-top)) if one_more else e / den


def latent_kv(h, W, p, m, eps):
    """What a latent attention caches: the normed latent [T, rank] and the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    d = lin(h, W, p + "dkv")
    c = rms_norm(d[:, :m["kv_rank"]], W[p + "dkv.norm"], eps)
    kr = rotate(d[:, m["kv_rank"]:].view(T, 1, m["rot_dim"]), m["rot"]).view(T, m["rot_dim"])
    return c, kr


def latent_attention(h, W, p, m, eps, shared=None, keep=None):
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_norm(lin(h, W, p + "dq"), W[p + "dq.norm"], eps)
    q = lin(cq, W, p + "uq").view(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate(q[..., dn:], m["rot"])
    c, kr = shared if shared is not None else latent_kv(h, W, p, m, eps)
    if keep is not None:
        keep["kv"] = (c, kr)
    kn = lin(c, W, p + "uk").view(T, H, dn)
    v = lin(c, W, p + "uv").view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    a = softmax_rows(s, visible(T, (m.get("mask") or {}).get("size")))
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * dv)
    return lin(o, W, p + "o")


def conv_attention(h, W, p, m, eps):
    """The left half of a parallel mixer: grouped heads, a short convolution behind each projection, a norm per
    head on q and k, a rotation of the leading elements, every earlier key, one more term in the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = lambda n: short_conv(lin(h, W, p + n), W[p + n + ".conv"])
    q = rms_norm(proj("q").view(T, H, d), W[p + "q.norm"], eps)
    k = rms_norm(proj("k").view(T, G, d), W[p + "k.norm"], eps)
    v = proj("v").view(T, G, dv)
    if m.get("rot"):
        q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    a = softmax_rows(s, visible(T, None), one_more=True)
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * dv)
    return lin(o, W, p + "o")


def matrix_memory(h, W, p, m, eps):
    """The right half: per head a matrix S [dim, vdim] and a vector n [dim] with a running maximum of the gates'
    logarithms."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (lin(h, W, p + "q") * d ** -0.5).view(T, H, d)
    k = lin(h, W, p + "k").view(T, H, d)
    v = lin(h, W, p + "v").view(T, H, dv)
    gi = cap * torch.tanh((lin(h, W, p + "i") + W[p + "i.b"].to(F)) / cap)
    gf = logsigmoid(cap * torch.tanh((lin(h, W, p + "f") + W[p + "f.b"].to(F)) / cap))
    S = torch.zeros(H, d, dv, dtype=F)
    n = torch.zeros(H, d, dtype=F)
    mx = torch.zeros(H, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, write = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + write[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + write[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = rms_norm(out, None, eps).reshape(T, H * dv) * W[p + "norm"].to(F)
    return lin(o * torch.sigmoid(lin(h, W, p + "g")), W, p + "o")


def parallel(h, W, p, m, eps):
    return (m["left_scale"] * conv_attention(h, W, p + "left.", m["left"], eps)
            + m["right_scale"] * matrix_memory(h, W, p + "right.", m["right"], eps))


def gated_recurrence(h, W, p, m):
    """Two branches of ``width``: a gate branch through gelu_tanh, and a convolved branch that feeds a linear
    recurrence per channel whose decay and input gate are logistic functions of block-diagonal products."""
    T = h.shape[0]
    C, B = m["width"], m["blocks"]
    y = gelu_tanh(lin(h, W, p + "y") + W[p + "y.b"].to(F))
    u = short_conv(lin(h, W, p + "x") + W[p + "x.b"].to(F), W[p + "conv"], W[p + "conv.b"])
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ra"].to(F)) + W[p + "ra.b"].to(F)).reshape(T, C)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, W[p + "ri"].to(F)) + W[p + "ri.b"].to(F)).reshape(T, C)
    a = torch.exp(-8.0 * r * softplus(W[p + "lam"].to(F)))
    S = torch.zeros(C, dtype=F)
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return lin(out * y, W, p + "o")


def dense(h, W, p):
    return lin(gelu_erf(lin(h, W, p + "up")), W, p + "down")


def route(z, r):
    """z [T, E] router logits -> (chosen experts [T, top], weights [T, top]): softmax over all experts, the best
    ``keep`` groups of neighbours by their largest score, the ``top`` largest scores among those, renormalised."""
    T, E = z.shape
    s = torch.softmax(z.to(F), dim=-1)
    groups = r.get("groups")
    allowed = torch.ones(T, E, dtype=torch.bool)
    if groups:
        per = E // groups["count"]
        best = s.view(T, groups["count"], per).max(-1).values
        kept = torch.topk(best, groups["keep"], dim=-1).indices
        allowed = torch.zeros(T, groups["count"], dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    chosen = torch.topk(masked, r["top"], dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20)


def experts(h, W, p, mlp):
    T = h.shape[0]
    chosen, w = route(lin(h, W, p + "router"), mlp["router"])
    out = torch.zeros(T, h.shape[1], dtype=F)
    for t in range(T):
        for e, we in zip(chosen[t].tolist(), w[t]):
            out[t] += we * dense(h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + dense(h, W, p + "shared.")
    return out


def forward(cfg, W, tokens, stream_after=None):
    """-> logits [T, vocab] (float64).  stream_after: a list that receives x after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"].to(F)[torch.tensor(tokens)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "latent_attention":
            kept[i] = {}
            shared = kept[m["kv_from"]]["kv"] if "kv_from" in m else None
            y = latent_attention(x, W, p, m, eps, shared, kept[i])
        elif layer["type"] == "parallel":
            y = parallel(x, W, p, m, eps)
        elif layer["type"] == "rglru":
            y = gated_recurrence(x, W, p, m)
        else:
            raise ValueError(layer["type"])
        x = rms_norm(alpha * x + y, W[f"l{i}.norm1"], eps, one_plus=True)
        mlp = layer.get("mlp")
        if mlp:
            y = dense(x, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else experts(x, W, f"l{i}.mlp.", mlp)
            x = rms_norm(alpha * x + y, W[f"l{i}.norm2"], eps, one_plus=True)
        if stream_after is not None:
            stream_after.append(x.clone())
    return rms_norm(x, W["final.norm"], eps, one_plus=True) @ W["embed"].to(F).T
