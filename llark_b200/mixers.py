"""Sequence mixers and feed-forwards of layer-list decoders on the generation path, by the `type` / `kind` names a
model's configuration uses. Each class packs its weights once (projections that read the same input become ONE matrix,
as the Llama path fuses q|k|v and gate|up), registers its per-request stores with the StateCache, and runs one packed
step through the C-ABI ops. Weights and state are separate objects: a layer that reuses another layer's weights gets
the same packed weights and stores of its own.

    "attention"  GatedWindowAttention   sliding-window softmax attention, per-head RMS norm of q and k, values = the
                                        un-normed keys, per-head temperature, sigmoid output gate
    "hgrn2"      GatedLinearRecurrence  HGRN2: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T silu(q)_t, forget
                                        gate with a learned lower bound, per-head RMS norm of o
    "dense"      ReluSquaredFF          down(relu(up x)^2)
"""
import torch

from . import ops

F32 = torch.float32


def _vec(w, name, dev):
    return w[name].to(device=dev, dtype=F32).contiguous()


def _mat(w, name, dev, act):
    return w[name].to(device=dev, dtype=act).contiguous()


class GatedWindowAttentionWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        G = int(spec.get("kv_heads", H))
        if H % G:
            raise ValueError("heads must be a multiple of kv_heads")
        if int(spec.get("vdim", D)) != D:
            raise ValueError("the values of this mixer are its keys: vdim must equal dim")
        self.H, self.G, self.D = H, G, D
        self.window = int(spec["mask"]["size"])
        # one projection for q | k | gate; the gate has no bias
        self.w_qkg = torch.cat([_mat(w, pfx + "q", dev, act), _mat(w, pfx + "k", dev, act), _mat(w, pfx + "g", dev, act)])
        self.b_qkg = torch.cat([_vec(w, pfx + "q.b", dev), _vec(w, pfx + "k.b", dev),
                                torch.zeros(H * D, device=dev, dtype=F32)])
        self.q_off, self.k_off, self.g_off = 0, H * D, (H + G) * D
        self.q_norm, self.k_norm = _vec(w, pfx + "q.norm", dev), _vec(w, pfx + "k.norm", dev)
        self.scale_h = (float(spec["scale"]) * _vec(w, pfx + "temp", dev)).contiguous()  # score scale per head
        self.w_o = _mat(w, pfx + "o", dev, act)
        for t, shape in ((self.w_qkg, ((2 * H + G) * D, width)), (self.w_o, (width, H * D)), (self.q_norm, (D,)),
                         (self.k_norm, (D,)), (self.scale_h, (H,))):
            if tuple(t.shape) != shape:
                raise ValueError(f"{pfx}: tensor of shape {tuple(t.shape)}, expected {shape}")


class GatedWindowAttention:
    Weights = GatedWindowAttentionWeights

    def __init__(self, weights, cache, eps, act, max_positions):
        self.w, self.eps, self.act = weights, float(eps), act
        w = weights
        self.cap = max(1, min(w.window, int(max_positions)))  # ring entries per request
        self.h_k = cache.add_store((self.cap, w.G * w.D), act, zero_on_alloc=False)
        self.h_v = cache.add_store((self.cap, w.G * w.D), act, zero_on_alloc=False)

    def forward(self, hc, st, cache):
        w = self.w
        kring, vring = cache.view(self.h_k), cache.view(self.h_v)
        qkg = ops.linear(hc, w.w_qkg, bias=w.b_qkg, out_dtype=F32)
        single = st.max_len == 1
        qn, kn, vr = ops.seq_qk_headnorm(qkg, w.q_off, w.k_off, w.q_norm, w.k_norm, w.H, w.G, w.D, self.eps, self.act,
                                         st=st, kring=kring if single else None, vring=vring if single else None,
                                         cap=self.cap)
        gate = qkg[:, w.g_off:]
        o = ops.seq_swa_attn(qn, kn, vr, kring, vring, gate, qkg.stride(0), w.scale_h, st, w.H, w.G, w.D, w.D,
                             w.window, self.cap, from_ring_only=single)
        if not single:
            ops.seq_kv_ring_write(kn, vr, kring, vring, st, self.cap)
        return ops.linear(o, w.w_o, out_dtype=F32)


class GatedLinearRecurrenceWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        H, D = int(spec["heads"]), int(spec["dim"])
        E = int(spec.get("vdim", D))
        self.H, self.D, self.E = H, D, E
        self.w_qfv = torch.cat([_mat(w, pfx + "q", dev, act), _mat(w, pfx + "f", dev, act), _mat(w, pfx + "v", dev, act)])
        self.b_qfv = torch.cat([torch.zeros(H * D, device=dev, dtype=F32), _vec(w, pfx + "f.b", dev),
                                torch.zeros(H * E, device=dev, dtype=F32)])
        self.q_off, self.f_off, self.v_off = 0, H * D, 2 * H * D
        self.lower = _vec(w, pfx + "lower", dev)
        self.norm = _vec(w, pfx + "norm", dev)
        self.w_o = _mat(w, pfx + "o", dev, act)
        for t, shape in ((self.w_qfv, (2 * H * D + H * E, width)), (self.w_o, (width, H * E)), (self.lower, (H * D,)),
                         (self.norm, (E,))):
            if tuple(t.shape) != shape:
                raise ValueError(f"{pfx}: tensor of shape {tuple(t.shape)}, expected {shape}")


class GatedLinearRecurrence:
    Weights = GatedLinearRecurrenceWeights

    def __init__(self, weights, cache, eps, act, max_positions):
        self.w, self.eps, self.act = weights, float(eps), act
        self.h_state = cache.add_store((weights.H, weights.D, weights.E), F32, zero_on_alloc=True)

    def forward(self, hc, st, cache):
        w = self.w
        qfv = ops.linear(hc, w.w_qfv, bias=w.b_qfv, out_dtype=F32)
        o_raw = ops.seq_glr_scan(qfv, w.q_off, w.f_off, w.v_off, w.lower, cache.view(self.h_state), st, w.H, w.D, w.E)
        o = ops.seq_head_rmsnorm(o_raw, w.norm, w.E, self.eps, self.act)
        return ops.linear(o, w.w_o, out_dtype=F32)


class ReluSquaredFFWeights:
    def __init__(self, w, pfx, spec, width, dev, act):
        F = int(spec["ff"])
        self.w_up, self.w_down = _mat(w, pfx + "up", dev, act), _mat(w, pfx + "down", dev, act)
        if tuple(self.w_up.shape) != (F, width) or tuple(self.w_down.shape) != (width, F):
            raise ValueError(f"{pfx}: feed-forward tensors do not fit ff = {F}")


class ReluSquaredFF:
    Weights = ReluSquaredFFWeights

    def __init__(self, weights, act):
        self.w, self.act = weights, act

    def forward(self, x_act):
        u = ops.linear(x_act, self.w.w_up, out_dtype=self.act)
        return ops.linear(ops.seq_relu2(u), self.w.w_down, out_dtype=F32)


MIXERS = {"attention": GatedWindowAttention, "hgrn2": GatedLinearRecurrence}
FEED_FORWARDS = {"dense": ReluSquaredFF}
