"""TEST INFRASTRUCTURE — second, independent restatement of the RWKV-7 forward step in numpy.

Used only by the test-suite: (1) to cross-check the C++ oracle (`rwkv7_cpu.cpp`) on small models, since
neither can be pinned against the Rust reference binary here, and (2) in float64, to adjudicate near-ties
when an arg-max token stream forks.  It is written from the algorithm as the reference's CPU path states it
(src/model.rs:396-517) but with vectorised numpy reductions, so its rounding differs from the C++ oracle's
and agreement is checked to a tolerance, not bit for bit.  Parity against the reference binary: unpinned.
"""
import numpy as np
from safetensors.numpy import load_file

LN_EPS, GN_EPS, L2_EPS = 1.0e-5, 64.0e-5, 1.0e-12


def dequant_int8(idx_u8, sz_u32):
    """w[m,k] = scale[m,k//128] * q + zero[m,k//128], fp32 (src/model.rs:234-252)."""
    scale = (sz_u32 & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    zero = (sz_u32 >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    return np.repeat(scale, 128, axis=1) * idx_u8.astype(np.float32) + np.repeat(zero, 128, axis=1)


class Rwkv7Numpy:
    def __init__(self, path, dtype=np.float64):
        t = load_file(path)
        self.dt = dtype
        f = lambda a: np.asarray(a, dtype=np.float32).astype(dtype)

        def linear(key):  # [out, in]
            if key in t:
                return f(t[key])
            return dequant_int8(t[key + ".int8_idx"], t[key + ".int8_sz"]).astype(dtype)

        self.V, self.C = t["emb.weight"].shape
        self.H, self.N = t["blocks.0.att.r_k"].shape
        self.L = 1 + max(int(k.split(".")[1]) for k in t if k.startswith("blocks."))
        self.emb = f(t["emb.weight"])
        self.ln0 = (f(t["blocks.0.ln0.weight"]), f(t["blocks.0.ln0.bias"]))
        self.ln_out = (f(t["ln_out.weight"]), f(t["ln_out.bias"]))
        self.head = linear("head.weight")
        C = self.C

        def lowrank(key, inp):  # -> [in, out]
            a = f(t[key])
            return a if a.shape[0] == inp and a.shape[1] != inp else a.T

        self.layers = []
        for i in range(self.L):
            p = f"blocks.{i}."
            g = lambda k: f(t[p + k]).reshape(-1)
            mids = {}
            lay = dict(
                ln1=(g("ln1.weight"), g("ln1.bias")), ln2=(g("ln2.weight"), g("ln2.bias")),
                ln_x=(g("att.ln_x.weight"), g("att.ln_x.bias")),
                x_r=g("att.x_r"), x_w=g("att.x_w"), x_k=g("att.x_k"), x_v=g("att.x_v"), x_a=g("att.x_a"), x_g=g("att.x_g"),
                w0=g("att.w0"), a0=g("att.a0"), v0=g("att.v0"), r_k=g("att.r_k"), k_k=g("att.k_k"), k_a=g("att.k_a"),
                ffn_x_k=g("ffn.x_k"),
                Wr=linear(p + "att.receptance.weight"), Wk=linear(p + "att.key.weight"), Wv=linear(p + "att.value.weight"),
                Wo=linear(p + "att.output.weight"), Wfk=linear(p + "ffn.key.weight"), Wfv=linear(p + "ffn.value.weight"),
            )
            for n in "wavg":
                m1 = f(t[p + f"att.{n}1"])
                mid = m1.shape[1] if m1.shape[0] == C else m1.shape[0]
                lay[n + "1"] = m1 if m1.shape == (C, mid) else m1.T          # [C, mid]
                m2 = f(t[p + f"att.{n}2"])
                lay[n + "2"] = m2 if m2.shape == (mid, C) else m2.T          # [mid, C]
            self.layers.append(lay)

    def new_state(self):
        z = lambda *s: np.zeros(s, dtype=self.dt)
        return [dict(tmix_x=z(self.C), S=z(self.H, self.N, self.N), cmix_x=z(self.C)) for _ in range(self.L)]

    @staticmethod
    def _ln(x, wb, eps):
        m = x.mean()
        v = ((x - m) ** 2).mean() + eps
        return (x - m) / np.sqrt(v) * wb[0] + wb[1]

    def forward_token(self, state, token):
        sig = lambda z: 1.0 / (1.0 + np.exp(-z))
        H, N = self.H, self.N
        x = self._ln(self.emb[token], self.ln0, LN_EPS)
        v_first = None
        for i, L in enumerate(self.layers):
            st = state[i]
            ln1 = self._ln(x, L["ln1"], LN_EPS)
            prev, st["tmix_x"] = st["tmix_x"], ln1
            mix = lambda m: ln1 + m * (prev - ln1)
            xr, xw, xk, xv, xa, xg = (mix(L[k]) for k in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g"))
            r, k, v = L["Wr"] @ xr, L["Wk"] @ xk, L["Wv"] @ xv
            if v_first is None:
                v_first = v
            else:
                v = v + sig(L["v0"] + (xv @ L["v1"]) @ L["v2"]) * (v_first - v)
            w = np.exp(-sig(L["w0"] + np.tanh(xw @ L["w1"]) @ L["w2"]) / np.sqrt(np.e))
            a = sig(L["a0"] + (xa @ L["a1"]) @ L["a2"])
            kk = (k * L["k_k"]).reshape(H, N)
            kk = kk / np.maximum(np.sqrt((kk * kk).sum(1, keepdims=True)), L2_EPS)
            k_mod = (k + L["k_a"] * (k * a - k)).reshape(H, N)
            b = -kk * a.reshape(H, N)
            S = st["S"]
            sa = np.einsum("hij,hj->hi", S, kk)
            S = S * w.reshape(H, 1, N) + sa[:, :, None] * b[:, None, :] + v.reshape(H, N)[:, :, None] * k_mod[:, None, :]
            st["S"] = S
            rh = r.reshape(H, N)
            y = np.einsum("hij,hj->hi", S, rh)
            m = y.mean(1, keepdims=True)
            var = ((y - m) ** 2).mean(1, keepdims=True) + GN_EPS
            y = ((y - m) / np.sqrt(var)).reshape(-1) * L["ln_x"][0] + L["ln_x"][1]
            bonus = (rh * k_mod * L["r_k"].reshape(H, N)).sum(1, keepdims=True) * v.reshape(H, N)
            y = y + bonus.reshape(-1)
            g = sig(xg @ L["g1"]) @ L["g2"]
            x = x + L["Wo"] @ (y * g)
            ln2 = self._ln(x, L["ln2"], LN_EPS)
            prev_c, st["cmix_x"] = st["cmix_x"], ln2
            xb = ln2 + L["ffn_x_k"] * (prev_c - ln2)
            x = x + L["Wfv"] @ (np.maximum(L["Wfk"] @ xb, 0.0) ** 2)
        self.last_hidden = x  # the last layer's residual stream, before ln_out
        return self.head @ self._ln(x, self.ln_out, LN_EPS)

    def forward(self, state, tokens):
        out = None
        for tok in tokens:
            out = self.forward_token(state, int(tok))
        return out
