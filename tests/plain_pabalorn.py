"""Pabalorn, plainly: every mechanism as one slow function in float64, written from the design's equations
and sharing nothing with the engine.  W maps tensor names to torch tensors; tokens is a list of ids.

Notation: x the residual stream [T, width]; N(w, y) = w * y / sqrt(mean(y^2) + eps) over the last axis;
N1(w, y) = N(1 + w, y) (a weight stored around zero).

    x = N1(w_e, embed[token])
    per layer: h = N1(w_1, x);  x <- x + mixer(h) + ff(h)        (one norm, both sublayers read it)
    logits = embed N1(w_f, x)
"""
import math

import torch

F = torch.float64


def rms_norm(y, w, eps, one_plus=False):
    y = y.to(F)
    w = w.to(F) + 1.0 if one_plus else w.to(F)
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def visible(T, window):
    """[T, T] true where query i sees key j: 0 <= i - j < window (window None: every earlier key)."""
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    return (d >= 0) & (d < window) if window else d >= 0


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` the wavelength rule: short waves kept, long ones
    divided by the factor, those between blended."""
    dims = rot["dims"]
    f = [rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f:
            wave = 2 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * fi / sc["factor"] + s * fi)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, rot, interleaved, first_position=0):
    """x [T, heads, d]: the first rot.dims elements of every head turned by position * f_i, pair i being
    (2i, 2i + 1) when interleaved and (i, i + dims/2) otherwise; the rest of the head unchanged."""
    if not rot:
        return x.to(F)
    x = x.to(F).clone()
    T, dims = x.shape[0], rot["dims"]
    half = dims // 2
    ang = (torch.arange(T, dtype=F) + first_position)[:, None] * rotary_frequencies(rot)[None, :]      # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    if interleaved:
        u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
        x[..., 0:dims:2] = u * c - v * s
        x[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :half].clone(), x[..., half:dims].clone()
        x[..., :half] = u * c - v * s
        x[..., half:dims] = v * c + u * s
    return x


def masked_softmax(s, mask):
    s = s.masked_fill(~mask, -math.inf)
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


def project_qkv(h, W, p, m, bias, interleaved, kv=True):
    """-> q [T, H, d] rotated, and (when kv) k [T, G, d] rotated, v [T, G, dv]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def lin(name):
        y = h.to(F) @ W[p + name].to(F).T
        return y + W[p + name + ".b"].to(F) if bias else y
    q = rotate(lin("q").view(T, H, d), m.get("rot"), interleaved)
    if not kv:
        return q, None, None
    return q, rotate(lin("k").view(T, G, d), m.get("rot"), interleaved), lin("v").view(T, G, dv)


def attend(q, k, v, m):
    """Scores q.k * scale, capped by a tanh when the mixer has a softcap, over the window; -> [T, H * dv]."""
    T, H = q.shape[0], m["heads"]
    rep = H // m["kv_heads"]
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    if m.get("softcap"):
        s = m["softcap"] * torch.tanh(s / m["softcap"])
    a = masked_softmax(s, visible(T, (m.get("mask") or {}).get("size")))
    return torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * m["vdim"])


def attention(h, W, p, m, bias=False, interleaved=False, shared_kv=None, keep=None):
    """An attention mixer whose tensors start with p.  shared_kv: (k, v) of the layer it takes them from;
    keep: a dict that receives this layer's (k, v) for such a layer."""
    q, k, v = project_qkv(h, W, p, m, bias, interleaved, kv=shared_kv is None)
    if shared_kv is not None:
        k, v = shared_kv
    if keep is not None:
        keep["kv"] = (k, v)
    return attend(q, k, v.to(F), m) @ W[p + "o"].to(F).T


def causal_conv(x, w, b):
    """x [T, C], w [C, taps] (last column: the current token's), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F), x.to(F)])
    y = sum(pad[j:j + T] * w[:, j].to(F) for j in range(taps))
    return y + b.to(F)


def selective_scan(h, W, p, m):
    """The recurrent mixer: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c."""
    T = h.shape[0]
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h.to(F) @ W[p + "in"].to(F).T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    dbc = x @ W[p + "x"].to(F).T
    dt = softplus(dbc[:, :R] @ W[p + "dt"].to(F).T + W[p + "dt.b"].to(F))          # [T, inner]
    B, Cm = dbc[:, R:R + N], dbc[:, R + N:R + 2 * N]
    A = -torch.exp(W[p + "A_log"].to(F))                                               # [inner, N]
    S = torch.zeros(inner, N, dtype=F)
    ys = []
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ Cm[t] + W[p + "D"].to(F) * x[t])
    y = torch.stack(ys) * silu(z)
    return y @ W[p + "o"].to(F).T


def side_by_side(h, W, p, m, eps):
    """Two mixers on the same input; half the sum of their outputs, each RMS-normed with a plain weight."""
    left = attention(h, W, p + "left.", m["left"], bias=True, interleaved=True)
    right = selective_scan(h, W, p + "right.", m["right"])
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


def expert(h, W, p):
    return (silu(h.to(F) @ W[p + "gate"].to(F).T) * (h.to(F) @ W[p + "up"].to(F).T)) @ W[p + "down"].to(F).T


def route(h, W, p, top):
    """-> (chosen experts [T, top], their weights [T, top]): the largest logistic scores, not renormalised."""
    s = torch.sigmoid(h.to(F) @ W[p + "router"].to(F).T)
    val, idx = s.topk(top, dim=-1)
    return idx, val


def routed_ff(h, W, p, m):
    """sum over the chosen experts of expert(w * h): the weight multiplies the expert's input."""
    idx, w = route(h, W, p, m["router"]["top"])
    out = torch.zeros(h.shape, dtype=F)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            out[t] += expert(w[t, c] * h[t:t + 1].to(F), W, p + f"e{int(idx[t, c])}.")[0]
    return out


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out, a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = rms_norm(W["embed"][torch.tensor(tokens)], W["embed.norm"], eps, one_plus=True)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps, one_plus=True)
        m = layer["mixer"]
        if layer["type"] == "attention":
            kept[i] = {}
            src = kept[m["kv_from"]]["kv"] if "kv_from" in m else None
            mixed = attention(h, W, p + "mix.", m, shared_kv=src, keep=kept[i])
        elif layer["type"] == "parallel":
            mixed = side_by_side(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            mixed = mixed + routed_ff(h, W, p + "mlp.", layer["mlp"])
        x = x + mixed
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps, one_plus=True) @ W["embed"].to(F).T
