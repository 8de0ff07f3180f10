"""CPU restatement (numpy) of the reference's ViT training step.

TEST INFRASTRUCTURE ONLY: this module is the checker for the CUDA path.  It is
imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline
legs, never by the library.

Every function restates one routine of the reference's CPU implementation and
cites it (paths are relative to the reference repository).  Array layouts are
the reference's: row-major, tokens as rows ``b*S + s``, attention rows as
``(b*H + h)*S + s``, weights ``[in, out]`` applied as ``X @ W``.

Pinning: tests/test_oracle_pinned.py checks this module against fixtures
produced by the reference's own compiled C code (oracle/_ref/libvithost.so,
built from the reference sources by oracle/build_ref.py; fixtures and the
script that wrote them live in tests/golden/), and against the closed-form
known answers of the reference's tests/test_vision.c.

All arithmetic runs in the dtype of the arrays passed in (float32 to mimic the
reference, float64 for a tighter yardstick); reductions use numpy's pairwise
summation, so results agree with the C loops to rounding, not bit for bit.
"""
import numpy as np

CLASSES_DEFAULT = 11
LAYER_NORM_EPSILON = 1e-5  # src/vit.c:494
ADAM_BETA1, ADAM_BETA2, ADAM_EPSILON = 0.9, 0.999, 1e-8  # src/vit.c:1085
CLIP_NORM = 1.0  # src/vit.c:1102


# --------------------------------------------------------------------- init

_MASK64 = (1 << 64) - 1


class SplitMix64:
    """src/vit.c:243-248."""

    def __init__(self, seed):
        self.state = seed & _MASK64

    def next(self):
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)

    def open_unit(self):
        """src/vit.c:250-252: ((x >> 40) + 0.5) / 2^24, in float32."""
        return (np.float32(self.next() >> 40) + np.float32(0.5)) / np.float32(16777216.0)

    def standard_normal(self):
        """src/vit.c:254-258 (Box-Muller, cosine branch)."""
        two_pi = np.float32(6.28318530717958647692)
        radius = np.sqrt(np.float32(-2.0) * np.log(self.open_unit()))
        return np.float32(radius * np.cos(two_pi * self.open_unit()))


def _xavier_uniform(rng, rows, cols):
    """src/vit.c:260-269."""
    limit = np.sqrt(np.float32(6.0) / (np.float32(rows) + np.float32(cols)))
    out = np.empty(rows * cols, dtype=np.float32)
    for i in range(out.size):
        out[i] = limit * (np.float32(2.0) * rng.open_unit() - np.float32(1.0))
    return out.reshape(rows, cols)


def _truncated_normal(rng, rows, cols, std):
    """src/vit.c:271-283: redraw while |z| > 2."""
    out = np.empty(rows * cols, dtype=np.float32)
    for i in range(out.size):
        z = rng.standard_normal()
        while abs(z) > 2.0:
            z = rng.standard_normal()
        out[i] = np.float32(std) * z
    return out.reshape(rows, cols)


def parameter_names(layers):
    """Optimiser order of the reference (src/vit.c:784-818)."""
    names = ["patch_projection", "patch_bias", "cls_token", "positional"]
    for layer in range(layers):
        names += [f"{layer}.{n}" for n in (
            "query_key_value", "query_key_value_bias", "attention_output",
            "attention_output_bias", "mlp_input", "mlp_input_bias",
            "mlp_output", "mlp_output_bias", "attention_gamma",
            "attention_beta", "mlp_gamma", "mlp_beta")]
    names += ["final_gamma", "final_beta", "head", "head_bias"]
    return names


def decays(name):
    """Weight decay applies to the six kinds of matrices only (src/vit.c:793-815)."""
    leaf = name.split(".")[-1]
    return leaf in ("patch_projection", "query_key_value", "attention_output",
                    "mlp_input", "mlp_output", "head")


def init_parameters(config, seed=42):
    """vit_model_init_seeded (src/vit.c:686-748): shapes, constants and the
    order in which the single random stream is consumed."""
    c, h, w, p, d, heads, layers, classes = config
    patches = (h // p) * (w // p)
    seq = patches + 1
    rng = SplitMix64(seed)
    params = {}
    params["patch_projection"] = _xavier_uniform(rng, c * p * p, d)
    params["patch_bias"] = np.zeros((1, d), np.float32)
    params["cls_token"] = _truncated_normal(rng, 1, d, 0.02)
    params["positional"] = _truncated_normal(rng, seq, d, 0.02)
    for layer in range(layers):
        k = f"{layer}."
        params[k + "query_key_value"] = _xavier_uniform(rng, d, 3 * d)
        params[k + "attention_output"] = _xavier_uniform(rng, d, d)
        params[k + "mlp_input"] = _xavier_uniform(rng, d, 4 * d)
        params[k + "mlp_output"] = _xavier_uniform(rng, 4 * d, d)
        params[k + "query_key_value_bias"] = np.zeros((1, 3 * d), np.float32)
        params[k + "attention_output_bias"] = np.zeros((1, d), np.float32)
        params[k + "mlp_input_bias"] = np.zeros((1, 4 * d), np.float32)
        params[k + "mlp_output_bias"] = np.zeros((1, d), np.float32)
        params[k + "attention_gamma"] = np.ones((1, d), np.float32)
        params[k + "attention_beta"] = np.zeros((1, d), np.float32)
        params[k + "mlp_gamma"] = np.ones((1, d), np.float32)
        params[k + "mlp_beta"] = np.zeros((1, d), np.float32)
    params["final_gamma"] = np.ones((1, d), np.float32)
    params["final_beta"] = np.zeros((1, d), np.float32)
    params["head"] = _truncated_normal(rng, d, classes, 0.02)
    params["head_bias"] = np.zeros((1, classes), np.float32)
    return {name: params[name] for name in parameter_names(layers)}


# ---------------------------------------------------------------- primitives

def gemm(x, w):
    """ops_gemm, src/ops.c:123-132."""
    return x @ w


def gemm_backward(x, w, dy):
    """ops_gemm_backward, src/ops.c:153-163: returns (dX, dW) increments."""
    return dy @ w.T, x.T @ dy


def extract_patches(images, c, h, w, p):
    """ops_extract_patches, src/ops.c:379-415: [B, C*H*W] -> [B*Np, C*P*P]."""
    b = images.shape[0]
    x = images.reshape(b, c, h // p, p, w // p, p)
    x = x.transpose(0, 2, 4, 1, 3, 5)  # b, py, px, c, y, x
    return np.ascontiguousarray(x).reshape(b * (h // p) * (w // p), c * p * p)


def extract_patches_backward(dpatches, b, c, h, w, p):
    """ops_extract_patches_backward, src/ops.c:417-432."""
    x = dpatches.reshape(b, h // p, w // p, c, p, p).transpose(0, 3, 1, 4, 2, 5)
    return np.ascontiguousarray(x).reshape(b, c * h * w)


def token_embedding(patch_tokens, cls, positional, batch):
    """ops_token_embedding, src/ops.c:450-480."""
    seq, d = positional.shape
    tokens = np.empty((batch, seq, d), patch_tokens.dtype)
    tokens[:, 0, :] = cls[0]
    tokens[:, 1:, :] = patch_tokens.reshape(batch, seq - 1, d)
    tokens += positional[None]
    return tokens.reshape(batch * seq, d)


def token_embedding_backward(dtokens, batch, seq):
    """ops_token_embedding_backward, src/ops.c:482-513:
    returns (d_patch_tokens, d_cls, d_positional)."""
    d = dtokens.shape[1]
    g = dtokens.reshape(batch, seq, d)
    return (np.ascontiguousarray(g[:, 1:, :]).reshape(batch * (seq - 1), d),
            g[:, 0, :].sum(axis=0, keepdims=True), g.sum(axis=0))


def layer_norm(x, gamma, beta, eps=LAYER_NORM_EPSILON):
    """ops_layer_norm, src/ops.c:773-815: two-pass mean / biased variance,
    1/sqrt(var + eps)."""
    dt = x.dtype.type
    mean = x.sum(axis=1, keepdims=True) / dt(x.shape[1])
    centred = x - mean
    var = (centred * centred).sum(axis=1, keepdims=True) / dt(x.shape[1])
    rstd = dt(1.0) / np.sqrt(var + dt(eps))
    return centred * rstd * gamma + beta


def layer_norm_backward(x, gamma, dy, eps=LAYER_NORM_EPSILON):
    """ops_layer_norm_backward, src/ops.c:845-904: returns (dx, dgamma, dbeta)."""
    dt = x.dtype.type
    n = dt(x.shape[1])
    mean = x.sum(axis=1, keepdims=True) / n
    centred = x - mean
    var = (centred * centred).sum(axis=1, keepdims=True) / n
    rstd = dt(1.0) / np.sqrt(var + dt(eps))
    xhat = centred * rstd
    dxhat = dy * gamma
    s1 = dxhat.sum(axis=1, keepdims=True)
    s2 = (dxhat * xhat).sum(axis=1, keepdims=True)
    dx = rstd * (dxhat - s1 / n - xhat * s2 / n)
    return dx, (dy * xhat).sum(axis=0, keepdims=True), dy.sum(axis=0, keepdims=True)


_GELU_C = 0.044715  # src/ops.c:944


def _gelu_scale(dt):
    """src/ops.c:946-948: sqrtf(2 / pi)."""
    return np.sqrt(dt(2.0) / dt(3.14159265358979323846))


def gelu(x):
    """ops_gelu, src/ops.c:956-964."""
    dt = x.dtype.type
    inner = _gelu_scale(dt) * (x + dt(_GELU_C) * x * x * x)
    return dt(0.5) * x * (dt(1.0) + np.tanh(inner))


def gelu_backward(x, dy):
    """ops_gelu_backward, src/ops.c:980-994."""
    dt = x.dtype.type
    s = _gelu_scale(dt)
    t = np.tanh(s * (x + dt(_GELU_C) * x * x * x))
    slope = dt(0.5) * (dt(1.0) + t) + dt(0.5) * x * (dt(1.0) - t * t) * s * (
        dt(1.0) + dt(3.0) * dt(_GELU_C) * x * x)
    return dy * slope


def split_heads(projected, batch, seq, d, heads):
    """ops_split_heads, src/ops.c:619-653: [R,3d] -> q,k,v [(b*H+h)*S+s, hd]."""
    hd = d // heads
    x = projected.reshape(batch, seq, 3, heads, hd).transpose(2, 0, 3, 1, 4)
    x = np.ascontiguousarray(x).reshape(3, batch * heads * seq, hd)
    return x[0], x[1], x[2]


def split_heads_backward(dq, dk, dv, batch, seq, d, heads):
    """ops_split_heads_backward, src/ops.c:655-691."""
    hd = d // heads
    x = np.stack([dq, dk, dv]).reshape(3, batch, heads, seq, hd)
    return np.ascontiguousarray(x.transpose(1, 3, 0, 2, 4)).reshape(batch * seq, 3 * d)


def merge_heads(attended, batch, seq, d, heads):
    """ops_merge_heads, src/ops.c:693-722."""
    hd = d // heads
    x = attended.reshape(batch, heads, seq, hd).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(x).reshape(batch * seq, d)


def merge_heads_backward(dmerged, batch, seq, d, heads):
    """ops_merge_heads_backward, src/ops.c:724-754."""
    hd = d // heads
    x = dmerged.reshape(batch, seq, heads, hd).transpose(0, 2, 1, 3)
    return np.ascontiguousarray(x).reshape(batch * heads * seq, hd)


def multi_head_attention(q, k, v, groups, seq, scale):
    """attention_forward_groups, src/ops.c:1297-1355: softmax over all keys
    (no mask), max-subtracted; returns (P [G*S, S], O [G*S, hd])."""
    hd = q.shape[1]
    dt = q.dtype.type
    qg, kg, vg = (t.reshape(groups, seq, hd) for t in (q, k, v))
    scores = np.matmul(qg, kg.transpose(0, 2, 1)) * dt(scale)
    scores = scores - scores.max(axis=2, keepdims=True)
    e = np.exp(scores)
    p = e / e.sum(axis=2, keepdims=True)
    o = np.matmul(p, vg)
    return p.reshape(groups * seq, seq), o.reshape(groups * seq, hd)


def multi_head_attention_backward(q, k, v, p, dout, groups, seq, scale):
    """attention_backward_groups, src/ops.c:1381-1441: returns (dq, dk, dv)."""
    hd = q.shape[1]
    dt = q.dtype.type
    qg, kg, vg, dog = (t.reshape(groups, seq, hd) for t in (q, k, v, dout))
    pg = p.reshape(groups, seq, seq)
    dv = np.matmul(pg.transpose(0, 2, 1), dog)
    dp = np.matmul(dog, vg.transpose(0, 2, 1))
    dot = (pg * dp).sum(axis=2, keepdims=True)
    ds = dt(scale) * pg * (dp - dot)
    dq = np.matmul(ds, kg)
    dk = np.matmul(ds.transpose(0, 2, 1), qg)
    return tuple(t.reshape(groups * seq, hd) for t in (dq, dk, dv))


def softmax_cross_entropy(logits, labels, class_weights=None, label_smoothing=0.0):
    """ops_softmax_cross_entropy_smoothed, src/ops.c:1025-1072:
    returns (loss, dlogits) with dlogits already divided by the row count."""
    dt = logits.dtype.type
    rows, cols = logits.shape
    off = dt(label_smoothing) / dt(cols)
    on = dt(1.0) - dt(label_smoothing) + off
    maximum = logits.max(axis=1, keepdims=True)
    lse = maximum + np.log(np.exp(logits - maximum).sum(axis=1, keepdims=True))
    target = np.full((rows, cols), off, logits.dtype)
    target[np.arange(rows), labels] = on
    weight = (np.ones((rows, 1), logits.dtype) if class_weights is None
              else np.asarray(class_weights, logits.dtype)[labels][:, None])
    loss = (weight * target * (lse - logits)).sum() / dt(rows)
    grad = weight * (np.exp(logits - lse) - target) / dt(rows)
    return dt(loss), grad


def clip_scale(grads, max_norm):
    """ops_clip_gradient_norm, src/ops.c:598-609: double-precision norm;
    scale only when norm > max_norm."""
    squared = 0.0
    for g in grads:
        squared += float((g.astype(np.float64) ** 2).sum())
    norm = np.sqrt(squared)
    if norm <= max_norm or norm == 0.0:
        return np.float32(1.0), norm
    return np.float32(max_norm / norm), norm


def adamw_update(w, g, m, v, step, lr, wd, beta1=ADAM_BETA1, beta2=ADAM_BETA2,
                 eps=ADAM_EPSILON):
    """apply_adamw_update, src/ops.c:1084-1100 (bias corrections by powf on the
    already-incremented step, src/ops.c:1080-1082).  Returns (w, m, v)."""
    dt = w.dtype.type
    c1 = dt(1.0) - np.power(dt(beta1), dt(step))
    c2 = dt(1.0) - np.power(dt(beta2), dt(step))
    m = dt(beta1) * m + (dt(1.0) - dt(beta1)) * g
    v = dt(beta2) * v + (dt(1.0) - dt(beta2)) * g * g
    estimate = (m / c1) / (np.sqrt(v / c2) + dt(eps))
    w = w - dt(lr) * (estimate + dt(wd) * w)
    return w, m, v


# -------------------------------------------------------------------- model

def forward(params, config, images):
    """vit_model_encode_forward + vit_encoder_block_forward_cached
    (src/vit.c:924-957, 483-538).  Returns (logits, cache)."""
    c, h, w, p, d, heads, layers, classes = config
    batch = images.shape[0]
    seq = (h // p) * (w // p) + 1
    dt = images.dtype.type
    cache = {"batch": batch, "seq": seq}
    cache["patches"] = extract_patches(images, c, h, w, p)
    patch_tokens = gemm(cache["patches"], params["patch_projection"]) + params["patch_bias"]
    x = token_embedding(patch_tokens, params["cls_token"], params["positional"], batch)
    cache["tokens"] = x
    scale = dt(1.0) / np.sqrt(dt(d // heads))
    for layer in range(layers):
        k = f"{layer}."
        blk = {"input": x}
        blk["normalized_attention"] = layer_norm(x, params[k + "attention_gamma"], params[k + "attention_beta"])
        blk["projected"] = gemm(blk["normalized_attention"], params[k + "query_key_value"]) + params[k + "query_key_value_bias"]
        blk["q"], blk["k"], blk["v"] = split_heads(blk["projected"], batch, seq, d, heads)
        blk["p"], blk["attended"] = multi_head_attention(blk["q"], blk["k"], blk["v"], batch * heads, seq, scale)
        blk["merged"] = merge_heads(blk["attended"], batch, seq, d, heads)
        branch = gemm(blk["merged"], params[k + "attention_output"]) + params[k + "attention_output_bias"]
        blk["attention_residual"] = x + branch
        blk["normalized_mlp"] = layer_norm(blk["attention_residual"], params[k + "mlp_gamma"], params[k + "mlp_beta"])
        blk["hidden"] = gemm(blk["normalized_mlp"], params[k + "mlp_input"]) + params[k + "mlp_input_bias"]
        blk["activated"] = gelu(blk["hidden"])
        mlp = gemm(blk["activated"], params[k + "mlp_output"]) + params[k + "mlp_output_bias"]
        x = blk["attention_residual"] + mlp
        blk["output"] = x
        cache[layer] = blk
    cache["normalized_tokens"] = layer_norm(x, params["final_gamma"], params["final_beta"])
    cache["cls_tokens"] = np.ascontiguousarray(cache["normalized_tokens"][::seq])  # ops_gather_rows, src/ops.c:515-532
    logits = gemm(cache["cls_tokens"], params["head"]) + params["head_bias"]
    return logits, cache


def backward(params, config, cache, dlogits):
    """vit_model_backward + vit_encoder_block_backward (src/vit.c:969-1013,
    540-599).  Returns the gradient of every parameter."""
    c, h, w, p, d, heads, layers, classes = config
    batch, seq = cache["batch"], cache["seq"]
    dt = dlogits.dtype.type
    scale = dt(1.0) / np.sqrt(dt(d // heads))
    grads = {}
    grads["head_bias"] = dlogits.sum(axis=0, keepdims=True)  # ops_bias_add_backward, src/ops.c:756-771
    dcls, grads["head"] = gemm_backward(cache["cls_tokens"], params["head"], dlogits)
    dnorm = np.zeros_like(cache["normalized_tokens"])
    dnorm[::seq] = dcls  # ops_gather_rows_backward, src/ops.c:534-552
    last = cache[layers - 1]["output"]
    dx, grads["final_gamma"], grads["final_beta"] = layer_norm_backward(last, params["final_gamma"], dnorm)
    for layer in reversed(range(layers)):
        k = f"{layer}."
        blk = cache[layer]
        # residual_backward: d(attention_residual) = d(mlp_branch) = dx
        grads[k + "mlp_output_bias"] = dx.sum(axis=0, keepdims=True)
        dact, grads[k + "mlp_output"] = gemm_backward(blk["activated"], params[k + "mlp_output"], dx)
        dhidden = gelu_backward(blk["hidden"], dact)
        grads[k + "mlp_input_bias"] = dhidden.sum(axis=0, keepdims=True)
        dnm, grads[k + "mlp_input"] = gemm_backward(blk["normalized_mlp"], params[k + "mlp_input"], dhidden)
        dres_ln, grads[k + "mlp_gamma"], grads[k + "mlp_beta"] = layer_norm_backward(
            blk["attention_residual"], params[k + "mlp_gamma"], dnm)
        dres = dx + dres_ln            # gradient of attention_residual
        grads[k + "attention_output_bias"] = dres.sum(axis=0, keepdims=True)
        dmerged, grads[k + "attention_output"] = gemm_backward(blk["merged"], params[k + "attention_output"], dres)
        dattended = merge_heads_backward(dmerged, batch, seq, d, heads)
        dq, dk, dv = multi_head_attention_backward(
            blk["q"], blk["k"], blk["v"], blk["p"], dattended, batch * heads, seq, scale)
        dproj = split_heads_backward(dq, dk, dv, batch, seq, d, heads)
        grads[k + "query_key_value_bias"] = dproj.sum(axis=0, keepdims=True)
        dna, grads[k + "query_key_value"] = gemm_backward(blk["normalized_attention"], params[k + "query_key_value"], dproj)
        dln, grads[k + "attention_gamma"], grads[k + "attention_beta"] = layer_norm_backward(
            blk["input"], params[k + "attention_gamma"], dna)
        dx = dres + dln                # accumulate_gradient(input, attention_residual) + LN
    dpatch, grads["cls_token"], grads["positional"] = token_embedding_backward(dx, batch, seq)
    grads["patch_bias"] = dpatch.sum(axis=0, keepdims=True)
    dpatches, grads["patch_projection"] = gemm_backward(cache["patches"], params["patch_projection"], dpatch)
    grads["__patches"] = dpatches
    return grads


def loss_and_gradients(params, config, images, labels, class_weights=None,
                       label_smoothing=0.0):
    """First half of vit_model_train_batch_smoothed (src/vit.c:1094-1112)."""
    logits, cache = forward(params, config, images)
    loss, dlogits = softmax_cross_entropy(logits, labels, class_weights, label_smoothing)
    grads = backward(params, config, cache, dlogits)
    grads.pop("__patches")
    return loss, grads, logits


class Trainer:
    """vit_model_train_batch_smoothed (src/vit.c:1094-1121) with its optimiser
    state: clip at 1.0, AdamW(0.9, 0.999, 1e-8), decay on matrices only."""

    def __init__(self, params, config):
        self.params = {k: v.copy() for k, v in params.items()}
        self.config = config
        self.m = {k: np.zeros_like(v) for k, v in params.items()}
        self.v = {k: np.zeros_like(v) for k, v in params.items()}
        self.step = 0

    def train_batch(self, images, labels, lr, weight_decay, class_weights=None,
                    label_smoothing=0.0):
        loss, grads, _ = loss_and_gradients(self.params, self.config, images, labels,
                                            class_weights, label_smoothing)
        names = parameter_names(self.config[6])
        self.step += 1  # src/ops.c:1140-1142
        scale, _ = clip_scale([grads[n] for n in names], CLIP_NORM)
        for n in names:
            g = grads[n] * grads[n].dtype.type(scale) if scale != 1.0 else grads[n]
            wd = weight_decay if decays(n) else 0.0
            self.params[n], self.m[n], self.v[n] = adamw_update(
                self.params[n], g, self.m[n], self.v[n], self.step, lr, wd)
        return loss
