"""Layer / model level restatement of the reference in numpy f64 on top of the C primitives.
TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Each function cites the reference lines it follows.  Items the reference does not have
(tanh, SiLU, causal masking, the plain multi-head block, a 16-action MLP policy) are marked
"extension": they are restated in the reference's style and are "parity unpinned".
"""
import math

import numpy as np

from . import (bias_add, bias_bwd, bmm_pv, bmm_pv_bwd, bmm_qkt, bmm_qkt_bwd, lcg_rand, linear_forward_inference,
               matmul, matmul_bwd, rmsnorm_bwd, rmsnorm_fwd, rope, rope_table, rope_token, softmax, softmax_bwd,
               softmax_exp_sum, vector_scale, dot_product, add_scaled_row)

# ------------------------------------------------------------------ activations


def act_fwd(z, kind):
    """relu: src/autograd.rs:356-361.  tanh / silu: extensions."""
    if kind in (None, "none"): return z
    if kind == "relu": return np.where(z > 0.0, z, 0.0)
    if kind == "tanh": return np.tanh(z)
    if kind == "silu": return z / (1.0 + np.exp(-z))
    raise ValueError(kind)


def act_bwd(g, z, y, kind):
    """dL/dz from dL/dy.  relu passes g where the INPUT is > 0 (src/autograd.rs:378-382)."""
    if kind in (None, "none"): return g
    if kind == "relu": return np.where(z > 0.0, g, 0.0)
    if kind == "tanh": return g * (1.0 - y * y)
    if kind == "silu":
        s = 1.0 / (1.0 + np.exp(-z)); return g * (s * (1.0 + z * (1.0 - s)))
    raise ValueError(kind)

# ------------------------------------------------------------------ Linear (src/nn.rs:12-142)


def linear_init_lcg(in_f, out_f, bias, seed):
    """Linear::new: Xavier limit sqrt(6/(in+out)) through the Tensor::rand LCG, bias zeros
    (src/nn.rs:20-35).  All weights come out negative (half-range LCG)."""
    limit = math.sqrt(6.0 / (in_f + out_f))
    W = lcg_rand((in_f, out_f), -limit, limit, seed)
    return W, (np.zeros(out_f) if bias else None)


def linear_fwd(x, W, b=None, threads=None):
    """Linear::forward (src/nn.rs:73-133): flatten leading dims, x.W, add bias per row."""
    shp = x.shape
    y = matmul(x.reshape(-1, W.shape[0]), W, threads)
    if b is not None: y = bias_add(y, b)
    return y.reshape(shp[:-1] + (W.shape[1],))


def linear_bwd(x, W, g, has_bias, threads=None, need_dx=True):
    x2 = x.reshape(-1, W.shape[0]); g2 = g.reshape(-1, W.shape[1])
    dx, dW = matmul_bwd(x2, W, g2, threads=threads, need_dA=need_dx)
    db = bias_bwd(g2, W.shape[1]) if has_bias else None
    return (dx.reshape(x.shape) if need_dx else None), dW, db

# ------------------------------------------------------------------ MLP (benchmark configuration 2; DQN-style placement, src/dqn.rs:70-74)


def mlp_fwd(X, Ws, bs, acts, threads=None):
    """Returns (pre-activations, activations) per layer."""
    zs, hs, h = [], [], X
    for W, b, a in zip(Ws, bs, acts):
        z = linear_fwd(h, W, b, threads); h = act_fwd(z, a); zs.append(z); hs.append(h)
    return zs, hs


def mlp_bwd(X, Ws, bs, acts, zs, hs, dY, threads=None, need_dx=True):
    dWs, dbs, g = [None] * len(Ws), [None] * len(Ws), dY
    for l in reversed(range(len(Ws))):
        g = act_bwd(g, zs[l], hs[l], acts[l])
        inp = X if l == 0 else hs[l - 1]
        g_in, dWs[l], dbs[l] = linear_bwd(inp, Ws[l], g, bs[l] is not None, threads, need_dx or l > 0)
        g = g_in
    return g, dWs, dbs

# ------------------------------------------------------------------ MLA (src/transformer.rs:375-1184)


class MLAConfig:
    def __init__(self, dim, num_heads, kv_lora_rank, qk_rope_dim, v_head_dim, max_seq_len):
        self.dim, self.num_heads, self.kv_lora_rank = dim, num_heads, kv_lora_rank
        self.qk_rope_dim, self.v_head_dim, self.max_seq_len = qk_rope_dim, v_head_dim, max_seq_len


def mla_init_lcg(cfg, seed):
    """MultiHeadLatentAttention::new seeds (src/transformer.rs:441-460), all bias-free."""
    full = cfg.num_heads * cfg.v_head_dim; hr = cfg.num_heads * cfg.qk_rope_dim
    shapes = [("dkv", cfg.dim, cfg.kv_lora_rank), ("uk", cfg.kv_lora_rank, full), ("uv", cfg.kv_lora_rank, full),
              ("q", cfg.dim, full), ("kr", cfg.dim, hr), ("qr", cfg.dim, hr), ("o", full, cfg.dim)]
    return {n: linear_init_lcg(i, o, False, seed + k)[0] for k, (n, i, o) in enumerate(shapes)}


def mla_forward(x, W, cfg, pos_mode="head_index", threads=None, return_cache=False):
    """MultiHeadLatentAttention::forward (src/transformer.rs:478-560).

    pos_mode "head_index" is the autograd path's actual behaviour: RoPE::forward rotates by
    the index along shape[-2] of a [B,S,H,dr] tensor, i.e. the head index (:262, :502-506).
    pos_mode "token" rotates by token position as the graph-free paths do (:583-610)."""
    B, S, D = x.shape; H, dh, dr = cfg.num_heads, cfg.v_head_dim, cfg.qk_rope_dim
    cosv, sinv = rope_table(dr, cfg.max_seq_len)
    x2 = x.reshape(B * S, D)
    c_kv = matmul(x2, W["dkv"], threads)
    k_c = matmul(c_kv, W["uk"], threads); v_c = matmul(c_kv, W["uv"], threads)
    k_r = matmul(x2, W["kr"], threads).reshape(B, S, H, dr)
    q_c = matmul(x2, W["q"], threads)
    q_r = matmul(x2, W["qr"], threads).reshape(B, S, H, dr)
    if pos_mode == "head_index":
        k_rot = rope(k_r, cosv, sinv, 0); q_rot = rope(q_r, cosv, sinv, 0)
    else:
        k_rot = rope_token(k_r, cosv, sinv, 0); q_rot = rope_token(q_r, cosv, sinv, 0)
    q = np.concatenate([q_c.reshape(B, S, H, dh), q_rot], axis=-1)      # concat_last_dim :1123
    k = np.concatenate([k_c.reshape(B, S, H, dh), k_rot], axis=-1)
    v = v_c.reshape(B, S, H, dh)
    qf = np.ascontiguousarray(q.swapaxes(1, 2)).reshape(B * H, S, dh + dr)   # transpose(1,2) + reshape :521-533
    kf = np.ascontiguousarray(k.swapaxes(1, 2)).reshape(B * H, S, dh + dr)
    vf = np.ascontiguousarray(v.swapaxes(1, 2)).reshape(B * H, S, dh)
    scores = bmm_qkt(qf, kf, threads) * (1.0 / math.sqrt(dh + dr))          # :539-543
    probs = softmax(scores)                                                  # non-causal :1074
    att = bmm_pv(probs, vf, threads)                                         # :549
    att = np.ascontiguousarray(att.reshape(B, H, S, dh).swapaxes(1, 2)).reshape(B * S, H * dh)
    out = matmul(att, W["o"], threads).reshape(B, S, D)
    if return_cache:
        return out, dict(x2=x2, c_kv=c_kv, qf=qf, kf=kf, vf=vf, probs=probs, att=att, cosv=cosv, sinv=sinv)
    return out


def mla_backward(g_out, W, cfg, cache, pos_mode="head_index", threads=None):
    """Backward of mla_forward, composed from the backward closures of the ops the forward
    calls (src/autograd.rs:268-351, src/transformer.rs:319-331, :920-955, :1010-1046,
    :1098-1117, :1162-1179).  Returns (dx, dW dict)."""
    H, dh, dr = cfg.num_heads, cfg.v_head_dim, cfg.qk_rope_dim
    x2 = cache["x2"]; BS, D = x2.shape; BH, S, _ = cache["qf"].shape; B = BH // H
    dW = {}
    d_att, dW["o"] = matmul_bwd(cache["att"], W["o"], g_out.reshape(BS, D), threads=threads)
    d_att = np.ascontiguousarray(d_att.reshape(B, S, H, dh).swapaxes(1, 2)).reshape(BH, S, dh)
    d_probs, d_vf = bmm_pv_bwd(cache["probs"], cache["vf"], d_att, threads)
    d_scores = softmax_bwd(cache["probs"], d_probs) * (1.0 / math.sqrt(dh + dr))
    d_qf, d_kf = bmm_qkt_bwd(cache["qf"], cache["kf"], d_scores, threads)

    def unflat(t, w):
        return np.ascontiguousarray(t.reshape(B, H, S, w).swapaxes(1, 2))      # [B,S,H,w]
    d_q = unflat(d_qf, dh + dr); d_k = unflat(d_kf, dh + dr); d_v = unflat(d_vf, dh)
    d_qc = np.ascontiguousarray(d_q[..., :dh]).reshape(BS, H * dh); d_qr = np.ascontiguousarray(d_q[..., dh:])
    d_kc = np.ascontiguousarray(d_k[..., :dh]).reshape(BS, H * dh); d_kr = np.ascontiguousarray(d_k[..., dh:])
    if pos_mode == "head_index":
        d_qr = rope(d_qr, cache["cosv"], cache["sinv"], 0, backward=True)
        d_kr = rope(d_kr, cache["cosv"], cache["sinv"], 0, backward=True)
    else:   # transposed rotation by token position == rotate by the negated angle
        d_qr = rope_token(d_qr, cache["cosv"], -cache["sinv"], 0)
        d_kr = rope_token(d_kr, cache["cosv"], -cache["sinv"], 0)
    dx = np.zeros_like(x2)
    d1, dW["qr"] = matmul_bwd(x2, W["qr"], d_qr.reshape(BS, H * dr), threads=threads); dx += d1
    d1, dW["q"] = matmul_bwd(x2, W["q"], d_qc, threads=threads); dx += d1
    d1, dW["kr"] = matmul_bwd(x2, W["kr"], d_kr.reshape(BS, H * dr), threads=threads); dx += d1
    d_ckv, dW["uv"] = matmul_bwd(cache["c_kv"], W["uv"], d_v.reshape(BS, H * dh), threads=threads)
    d2, dW["uk"] = matmul_bwd(cache["c_kv"], W["uk"], d_kc, threads=threads); d_ckv += d2
    d1, dW["dkv"] = matmul_bwd(x2, W["dkv"], d_ckv, threads=threads); dx += d1
    return dx.reshape(B, S, D), dW


class KVCache:
    """src/transformer.rs:400-425: per-head growing K ([len, dh+dr]) and V ([len, dh]) rows."""

    def __init__(self, num_heads):
        self.k = [np.zeros((0,)) for _ in range(num_heads)]
        self.v = [np.zeros((0,)) for _ in range(num_heads)]


def mla_forward_inference_cached(x, W, cfg, cache, start_pos):
    """forward_inference_cached (src/transformer.rs:688-841): graph-free path over one or a
    few tokens, token-position RoPE, K/V appended to the cache, softmax over all cached rows."""
    D, H, dh, dr = cfg.dim, cfg.num_heads, cfg.v_head_dim, cfg.qk_rope_dim
    S = x.size // D; tot = dh + dr
    cosv, sinv = rope_table(dr, cfg.max_seq_len)
    lin = linear_forward_inference
    c_kv = lin(x, W["dkv"]); k_c = lin(c_kv, W["uk"]); v_c = lin(c_kv, W["uv"])
    k_r = lin(x, W["kr"]); q_c = lin(x, W["q"]); q_r = lin(x, W["qr"])
    k_rot = rope_token(k_r.reshape(1, S, H, dr), cosv, sinv, start_pos).reshape(S, H, dr)
    q_rot = rope_token(q_r.reshape(1, S, H, dr), cosv, sinv, start_pos).reshape(S, H, dr)
    q = np.concatenate([q_c.reshape(S, H, dh), q_rot], axis=-1)
    k = np.concatenate([k_c.reshape(S, H, dh), k_rot], axis=-1)
    v = v_c.reshape(S, H, dh)
    for t in range(S):
        for h in range(H):
            cache.k[h] = np.concatenate([cache.k[h], k[t, h]]); cache.v[h] = np.concatenate([cache.v[h], v[t, h]])
    L = cache.k[0].size // tot; scale = 1.0 / math.sqrt(tot)
    att_out = np.zeros((S, H, dh))
    for h in range(H):
        kc = cache.k[h].reshape(L, tot); vc = cache.v[h].reshape(L, dh)
        for i in range(S):
            sc = np.array([dot_product(q[i, h], kc[j]) * scale for j in range(L)])
            e, s = softmax_exp_sum(sc); p = vector_scale(e, 1.0 / s)
            o = np.zeros(dh)
            for j in range(L):
                if abs(p[j]) < 1e-9: continue                     # :830-832
                o = add_scaled_row(o, vc[j], p[j])
            att_out[i, h] = o
    return lin(att_out.reshape(-1), W["o"])


def prune_kv_cache(cache, cfg, max_seq_len):
    """prune_kv_cache (src/transformer.rs:843-874): drop the oldest rows beyond max_seq_len."""
    tot = cfg.v_head_dim + cfg.qk_rope_dim
    cur = cache.k[0].size // tot
    if cur > max_seq_len:
        rm = cur - max_seq_len
        for h in range(len(cache.k)):
            cache.k[h] = cache.k[h][rm * tot:]; cache.v[h] = cache.v[h][rm * cfg.v_head_dim:]

# ------------------------------------------------------------------ LuckTransformer / ActorCritic (reference's own block)


class LuckTransformer:
    """src/transformer.rs:36-216: embed -> norm_1 -> MLA -> +res -> norm_2 -> FFN(ReLU, 2x) -> +res
    -> norm_final -> out_proj; RMSNorm eps 1e-5; heads 4, latent 32, rope 16, dv hidden/4."""

    def __init__(self, in_dim, hidden, seed):
        self.cfg = MLAConfig(hidden, 4, 32, 16, hidden // 4, 256)
        self.embed = linear_init_lcg(in_dim, hidden, True, seed)
        self.mla = mla_init_lcg(self.cfg, seed + 10)
        self.ffn_1 = linear_init_lcg(hidden, hidden * 2, True, seed + 20)
        self.ffn_2 = linear_init_lcg(hidden * 2, hidden, True, seed + 30)
        self.out_proj = linear_init_lcg(hidden, hidden, True, seed + 40)
        self.g1 = np.ones(hidden); self.g2 = np.ones(hidden); self.gf = np.ones(hidden)
        self.eps = 1e-5

    def forward(self, x, pos_mode="head_index"):
        """Autograd-path forward (:71-90) on [B,S,in]."""
        h = linear_fwd(x, *self.embed)
        n1 = rmsnorm_fwd(h, self.g1, self.eps)[0]
        h2 = h + mla_forward(n1, self.mla, self.cfg, pos_mode)
        n2 = rmsnorm_fwd(h2, self.g2, self.eps)[0]
        f1 = act_fwd(linear_fwd(n2, *self.ffn_1), "relu")
        h3 = h2 + linear_fwd(f1, *self.ffn_2)
        return linear_fwd(rmsnorm_fwd(h3, self.gf, self.eps)[0], *self.out_proj)

    def forward_backward(self, x, g_out, pos_mode="head_index"):
        """Forward (:71-90) and the backward the tape would run.  Returns (output, dx, grads) with grads in
        LuckTransformer::parameters order (:205-215): embed W,b; norm_1; MLA dkv,uk,uv,q,kr,qr,o; norm_2;
        ffn_1 W,b; ffn_2 W,b; norm_final; out_proj W,b."""
        B, S, _ = x.shape
        h = linear_fwd(x, *self.embed)
        n1, rms1, xh1 = rmsnorm_fwd(h, self.g1, self.eps)
        att, cache = mla_forward(n1, self.mla, self.cfg, pos_mode, return_cache=True)
        h2 = h + att
        n2, rms2, xh2 = rmsnorm_fwd(h2, self.g2, self.eps)
        z1 = linear_fwd(n2, *self.ffn_1); f1 = act_fwd(z1, "relu")
        h3 = h2 + linear_fwd(f1, *self.ffn_2)
        nf, rmsf, xhf = rmsnorm_fwd(h3, self.gf, self.eps)
        out = linear_fwd(nf, *self.out_proj)
        d_nf, dWo, dbo = linear_bwd(nf, self.out_proj[0], g_out, True)
        d_h3, dgf = rmsnorm_bwd(d_nf, self.gf, rmsf, xhf)
        d_f1, dW2, db2 = linear_bwd(f1, self.ffn_2[0], d_h3, True)
        d_z1 = act_bwd(d_f1, z1, f1, "relu")
        d_n2, dW1, db1 = linear_bwd(n2, self.ffn_1[0], d_z1, True)
        d_h2, dg2 = rmsnorm_bwd(d_n2, self.g2, rms2, xh2); d_h2 = d_h2 + d_h3
        d_n1, dmla = mla_backward(d_h2, self.mla, self.cfg, cache, pos_mode)
        d_h, dg1 = rmsnorm_bwd(d_n1, self.g1, rms1, xh1); d_h = d_h + d_h2
        dx, dWe, dbe = linear_bwd(x, self.embed[0], d_h, True)
        grads = [dWe, dbe, dg1] + [dmla[k] for k in ("dkv", "uk", "uv", "q", "kr", "qr", "o")] + [dg2, dW1, db1, dW2, db2, dgf, dWo, dbo]
        return out, dx, grads

    def forward_inference_step(self, x, cache, start_pos):
        """forward_inference_step (:152-193): one token through the KV-cached path."""
        lin = linear_forward_inference

        def norm(v, g):
            return rmsnorm_fwd(v, g, self.eps)[0]      # RMSNorm::forward_inference has the same arithmetic (src/nn.rs:160-179)
        h = lin(x, *self.embed)
        h2 = h + mla_forward_inference_cached(norm(h, self.g1), self.mla, self.cfg, cache, start_pos)
        f1 = lin(norm(h2, self.g2), *self.ffn_1); f1 = np.where(f1 < 0.0, 0.0, f1)
        h3 = h2 + lin(f1, *self.ffn_2)
        return lin(norm(h3, self.gf), *self.out_proj)


class ActorCritic:
    """src/ppo.rs:247-307: LuckTransformer(8, 64) + actor head 64->5 (seed+100) + critic 64->1 (seed+200)."""

    def __init__(self, seed, in_dim=8, hidden=64, actions=5):
        self.backbone = LuckTransformer(in_dim, hidden, seed)
        self.actor = linear_init_lcg(hidden, actions, True, seed + 100)
        self.critic = linear_init_lcg(hidden, 1, True, seed + 200)

    def forward_actor(self, state, pos_mode="head_index"):
        x = state.reshape((1, 1, -1)) if state.ndim == 1 else state.reshape((1,) + state.shape) if state.ndim == 2 else state
        seq = self.backbone.forward(x, pos_mode)
        last = seq[:, -1, :]                                   # last_token :92-109
        return linear_fwd(last, *self.actor).reshape(-1)

    def step_probs_inference_cached(self, state, cache, start_pos):
        """The deterministic part of step_inference_cached (src/ppo.rs:391-412): one token through the KV-cached
        backbone, actor head, softmax with max subtraction.  (The sampling that follows uses rand::random and is
        outside parity.)"""
        last = self.backbone.forward_inference_step(state, cache, start_pos)
        logits = linear_forward_inference(last, *self.actor)
        e = np.exp(logits - logits.max())
        return e / e.sum()


def rollout_reference(ac, states, resets, context_len):
    """What the simulator does with the cached policy for each of N simulations independently
    (src/sim.rs:208, :578, :171-175): step t calls step_inference_cached(state, cache, start_pos = pulls done
    in this episode), then prunes the cache to `context_len`; resets[t, n] != 0 ends simulation n's episode
    after step t (fresh KVCache, start_pos back to 0).  states [T, N, in]; returns probabilities [T, N, A]."""
    T, N, _ = states.shape
    caches = [KVCache(ac.backbone.cfg.num_heads) for _ in range(N)]
    pos = [0] * N
    out = []
    for t in range(T):
        row = []
        for n in range(N):
            row.append(ac.step_probs_inference_cached(states[t, n], caches[n], pos[n]))
            prune_kv_cache(caches[n], ac.backbone.cfg, context_len)
            if resets[t, n]:
                caches[n] = KVCache(ac.backbone.cfg.num_heads); pos[n] = 0
            else:
                pos[n] += 1
        out.append(row)
    return np.array(out)

# ------------------------------------------------------------------ dueling double-DQN pieces (src/dqn.rs)


def dueling_combine(v, adv):
    """DuelingQNetwork::forward_impl, batch branch (src/dqn.rs:76-93): val.ones(1,A) + adv - (adv.ones(A,1)/A).ones(1,A)."""
    A = adv.shape[1]
    return v.reshape(-1, 1) @ np.ones((1, A)) + adv - (adv @ np.full((A, 1), 1.0 / A)) @ np.ones((1, A))


def dueling_combine_bwd(dq):
    """Backward of the three matmuls: dv = dq.ones(A,1); dadv = dq - (dq.ones(A,1)).(ones(1,A)/A)."""
    A = dq.shape[1]
    dv = dq @ np.ones((A, 1))
    return dv, dq - dv @ np.full((1, A), 1.0 / A)


def dqn_target(q_next_eval, q_next_target, rewards, dones, gamma=0.99):
    """src/dqn.rs:524-556: argmax (first maximum) from the online network, value from the target network."""
    out = np.empty(len(rewards))
    for i in range(len(rewards)):
        best, mx = 0, -np.inf
        for k, val in enumerate(q_next_eval[i]):
            if val > mx:
                mx, best = val, k
        out[i] = rewards[i] + gamma * q_next_target[i, best] * (1.0 - dones[i])
    return out


def dqn_loss_fwd_bwd(q, actions, target):
    """(q * mask).ones(A,1) then mse_loss (src/dqn.rs:516-561, src/autograd.rs:1599-1603) and its gradient w.r.t. q."""
    B = q.shape[0]
    sel = q[np.arange(B), actions]
    d = sel - target
    dq = np.zeros_like(q); dq[np.arange(B), actions] = 2.0 * d / B
    return float(np.mean(d * d)), dq


def soft_update(target, source, tau):
    """src/dqn.rs:129-150."""
    return target * (1.0 - tau) + source * tau

# ------------------------------------------------------------------ plain multi-head block (benchmark configuration 3) -- extension


def block_fwd(x, P, heads, eps=1e-6, threads=None):
    """Pre-norm block in the reference's residual order (src/transformer.rs:71-90) with the
    config-3 contents: RMSNorm -> QKV -> RoPE(token positions, whole head, interleaved pairs)
    -> causal softmax attention, scale 1/sqrt(dh) -> W_o -> +res -> RMSNorm -> W_ff1 -> SiLU ->
    W_ff2 -> +res.  No biases.  Returns (y, cache)."""
    B, S, D = x.shape; dh = D // heads
    cosv, sinv = rope_table(dh, S)
    x2 = x.reshape(B * S, D)
    n1, rms1, xh1 = rmsnorm_fwd(x2, P["g1"], eps)
    qkv = matmul(n1, P["w_qkv"], threads).reshape(B, S, 3, heads, dh)
    q = rope_token(np.ascontiguousarray(qkv[:, :, 0]), cosv, sinv)
    k = rope_token(np.ascontiguousarray(qkv[:, :, 1]), cosv, sinv)
    v = np.ascontiguousarray(qkv[:, :, 2])
    qf = np.ascontiguousarray(q.swapaxes(1, 2)).reshape(B * heads, S, dh)
    kf = np.ascontiguousarray(k.swapaxes(1, 2)).reshape(B * heads, S, dh)
    vf = np.ascontiguousarray(v.swapaxes(1, 2)).reshape(B * heads, S, dh)
    scores = bmm_qkt(qf, kf, threads) * (1.0 / math.sqrt(dh))
    probs = softmax(scores, causal_period=S)
    att = bmm_pv(probs, vf, threads)
    att2 = np.ascontiguousarray(att.reshape(B, heads, S, dh).swapaxes(1, 2)).reshape(B * S, D)
    h2 = x2 + matmul(att2, P["w_o"], threads)
    n2, rms2, xh2 = rmsnorm_fwd(h2, P["g2"], eps)
    z = matmul(n2, P["w_ff1"], threads); f = act_fwd(z, "silu")
    y = h2 + matmul(f, P["w_ff2"], threads)
    cache = dict(x2=x2, n1=n1, rms1=rms1, xh1=xh1, qf=qf, kf=kf, vf=vf, probs=probs, att2=att2, h2=h2,
                 n2=n2, rms2=rms2, xh2=xh2, z=z, f=f, cosv=cosv, sinv=sinv, shape=(B, S, D, heads, dh))
    return y.reshape(B, S, D), cache


def block_bwd(g, P, cache, threads=None):
    B, S, D, heads, dh = cache["shape"]; g2 = g.reshape(B * S, D); dP = {}
    d_f, dP["w_ff2"] = matmul_bwd(cache["f"], P["w_ff2"], g2, threads=threads)
    d_z = act_bwd(d_f, cache["z"], cache["f"], "silu")
    d_n2, dP["w_ff1"] = matmul_bwd(cache["n2"], P["w_ff1"], d_z, threads=threads)
    d_h2, dP["g2"] = rmsnorm_bwd(d_n2, P["g2"], cache["rms2"], cache["xh2"]); d_h2 += g2
    d_att2, dP["w_o"] = matmul_bwd(cache["att2"], P["w_o"], d_h2, threads=threads)
    d_att = np.ascontiguousarray(d_att2.reshape(B, S, heads, dh).swapaxes(1, 2)).reshape(B * heads, S, dh)
    d_probs, d_vf = bmm_pv_bwd(cache["probs"], cache["vf"], d_att, threads)
    d_scores = softmax_bwd(cache["probs"], d_probs) * (1.0 / math.sqrt(dh))
    d_qf, d_kf = bmm_qkt_bwd(cache["qf"], cache["kf"], d_scores, threads)

    def unflat(t):
        return np.ascontiguousarray(t.reshape(B, heads, S, dh).swapaxes(1, 2))
    d_q = rope_token(unflat(d_qf), cache["cosv"], -cache["sinv"])
    d_k = rope_token(unflat(d_kf), cache["cosv"], -cache["sinv"])
    d_qkv = np.stack([d_q, d_k, unflat(d_vf)], axis=2).reshape(B * S, 3 * D)
    d_n1, dP["w_qkv"] = matmul_bwd(cache["n1"], P["w_qkv"], d_qkv, threads=threads)
    d_x, dP["g1"] = rmsnorm_bwd(d_n1, P["g1"], cache["rms1"], cache["xh1"]); d_x += d_h2
    return d_x.reshape(B, S, D), dP

# ------------------------------------------------------------------ PPO (src/ppo.rs)

CLIP_EPSILON, VALUE_COEF, ENTROPY_COEF = 0.2, 0.5, 0.01      # src/ppo.rs:17-21


def ppo_loss_fwd_bwd(logits, values, actions, old_logp, adv, ret, clip=CLIP_EPSILON, c_v=VALUE_COEF,
                     c_h=ENTROPY_COEF, denom=None):
    """The per-sample loss of PPO::update (src/ppo.rs:702-755), vectorised over the minibatch.

    logp = logits - logsumexp (max-subtracted, :702-718); ratio = exp(logp[a] - old) (:720-725);
    kl = (ratio-1) - log_ratio (:729); surr1 = ratio*A, surr2 = clip(ratio)*A, surr1 is used iff
    surr1 < surr2 (:734-740); clip passes gradient iff 0.8 <= ratio <= 1.2 inclusive
    (src/autograd.rs:761); v_loss = (v-R)^2 (:743); H = -sum p*logp (:745-746);
    loss = -policy + c_v*v_loss - c_h*H, averaged over the minibatch (:748-755).
    Returns (mean loss, dL/dlogits, dL/dvalues, sum of kl)."""
    n, A = logits.shape; denom = float(n if denom is None else denom)
    mx = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - mx).sum(axis=1, keepdims=True)) + mx
    logp = logits - lse; p = np.exp(logp)
    idx = np.arange(n)
    lp_a = logp[idx, actions]; log_ratio = lp_a - old_logp; ratio = np.exp(log_ratio)
    kl = (ratio - 1.0) - log_ratio
    surr1 = ratio * adv; surr2 = np.clip(ratio, 1.0 - clip, 1.0 + clip) * adv
    use1 = surr1 < surr2
    policy = np.where(use1, surr1, surr2)
    v_loss = (values - ret) ** 2
    ent = -(p * logp).sum(axis=1)
    loss = (-policy + c_v * v_loss - c_h * ent).sum() / denom
    inside = (ratio >= 1.0 - clip) & (ratio <= 1.0 + clip)
    d_ratio = np.where(use1, adv, np.where(inside, adv, 0.0))
    d_lp_a = -(d_ratio * ratio)                                 # d(-policy)/d logp[a]
    d_logp = c_h * p * (logp + 1.0)                             # d(-c_h*H)/d logp_j = c_h p_j (logp_j + 1)
    d_logp[idx, actions] += d_lp_a
    d_logits = d_logp - p * d_logp.sum(axis=1, keepdims=True)   # logp = logits - lse, d lse/d logits = p
    d_values = c_v * 2.0 * (values - ret)
    return loss, d_logits / denom, d_values / denom, kl.sum()


def adam_step(params, grads, m, v, t, lr, b1=0.9, b2=0.999, eps=1e-8, clip_norm=None):
    """Adam::step (src/ppo.rs:519-533); clip_norm=1.0 gives the DQN variant with global-norm
    clipping (src/dqn.rs:207-239).  `t` is the step count AFTER the increment.  In place."""
    coef = 1.0
    if clip_norm is not None:
        total = math.sqrt(sum(float((g * g).sum()) for g in grads))
        coef = clip_norm / total if total > clip_norm else 1.0
    for p, g, mi, vi in zip(params, grads, m, v):
        g = g * coef
        mi *= b1; mi += (1.0 - b1) * g
        vi *= b2; vi += (1.0 - b2) * g * g
        m_hat = mi / (1.0 - b1 ** t); v_hat = vi / (1.0 - b2 ** t)
        p -= lr * m_hat / (np.sqrt(v_hat) + eps)


class MlpActorCritic:
    """benchmark configuration 5 policy (extension): trunk obs->h->h with tanh, policy head h->A, value
    head h->1, the ActorCritic split of src/ppo.rs:247-307 on an MLP trunk."""
    NAMES = ["w1", "b1", "w2", "b2", "wp", "bp", "wv", "bv"]

    def __init__(self, params):
        self.p = {k: np.array(params[k], dtype=np.float64) for k in self.NAMES}

    def forward(self, obs, threads=None):
        p = self.p
        zs, hs = mlp_fwd(obs, [p["w1"], p["w2"]], [p["b1"], p["b2"]], ["tanh", "tanh"], threads)
        logits = linear_fwd(hs[1], p["wp"], p["bp"], threads)
        values = linear_fwd(hs[1], p["wv"], p["bv"], threads).reshape(-1)
        return zs, hs, logits, values

    def grads(self, obs, actions, old_logp, adv, ret, threads=None, denom=None):
        """Minibatch gradient of the PPO loss; returns (grad dict, loss, kl sum)."""
        p = self.p
        zs, hs, logits, values = self.forward(obs, threads)
        loss, dl, dv, kl = ppo_loss_fwd_bwd(logits, values, actions, old_logp, adv, ret, denom=denom)
        g = {}
        dh_p, g["wp"], g["bp"] = linear_bwd(hs[1], p["wp"], dl, True, threads)
        dh_v, g["wv"], g["bv"] = linear_bwd(hs[1], p["wv"], dv.reshape(-1, 1), True, threads)
        _, dWs, dbs = mlp_bwd(obs, [p["w1"], p["w2"]], [p["b1"], p["b2"]], ["tanh", "tanh"], zs, hs, dh_p + dh_v,
                              threads, need_dx=False)
        g["w1"], g["w2"], g["b1"], g["b2"] = dWs[0], dWs[1], dbs[0], dbs[1]
        return g, loss, kl

    def log_prob(self, obs, actions, threads=None):
        _, _, logits, _ = self.forward(obs, threads)
        mx = logits.max(axis=1, keepdims=True)
        logp = logits - (np.log(np.exp(logits - mx).sum(axis=1, keepdims=True)) + mx)
        return logp[np.arange(len(actions)), actions]


def ppo_update(model, obs, actions, old_logp, adv, ret, epochs, minibatch, lr=3e-4, kl_stop=None, threads=None,
               opt=None):
    """PPO::update's optimisation loops (src/ppo.rs:680-769): consecutive unshuffled minibatches,
    zero_grad -> mean loss -> backward -> Adam step, per-epoch mean KL with optional early stop
    at 1.5 * target (kl_stop = 0.015 reproduces :678, :764).  Returns per-epoch mean KL."""
    names = model.NAMES
    if opt is None:
        opt = dict(m=[np.zeros_like(model.p[k]) for k in names], v=[np.zeros_like(model.p[k]) for k in names], t=0)
    kls = []
    n = obs.shape[0]
    for _ in range(epochs):
        kl_sum, cnt = 0.0, 0
        for s in range(0, n, minibatch):
            e = min(n, s + minibatch)
            g, _, kl = model.grads(obs[s:e], actions[s:e], old_logp[s:e], adv[s:e], ret[s:e], threads)
            kl_sum += kl; cnt += e - s
            opt["t"] += 1
            adam_step([model.p[k] for k in names], [g[k] for k in names], opt["m"], opt["v"], opt["t"], lr)
        kls.append(kl_sum / cnt)
        if kl_stop is not None and kls[-1] > kl_stop * 1.5: break
    return kls, opt
