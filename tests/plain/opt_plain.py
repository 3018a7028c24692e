"""Plain, slow implementation of the OPT decoder used as the oracle of every test.

Each function below is written from a formula of aws-neuron/transformers-neuronx and cites its
place, by the file's path within that project (``T/`` = ``src/transformers_neuronx/``).  That
project states the model only as Python that builds an HLO graph for the Neuron compiler (its
``OPTDecoderLayer`` in ``T/opt/model.py:247-257`` has no forward method), so its model cannot be
compiled or run as it is here.  Its graph-building code, however, is ordinary Python:
tests/golden/reference_graph_eager.py runs the reference's own layer, attention, LayerNorm and head
functions operation by operation on the CPU, and tests/test_golden.py compares this file with the
logits that came out (a left-padded batch at every prompt position and three decode steps; 2e-5).
What else of the reference runs on the CPU (the checkpoint writer's tensor names and shapes, the
top-k / top-p filter) is pinned by the other files of tests/golden/.

Whole sequences, no cache, one function for each part, plain torch on the CPU in
32-bit (or 64-bit) floats.  It shares no code with the engine: it reads a
``{name: tensor}`` dictionary and a plain ``dict`` of config.json keys.

Where the reference has no formula (post-LN placement, project_in/project_out,
switches for bias and LayerNorm affine) the function says so and states the
convention that the engine follows.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

# Constants fixed in the reference's code, not in config.json.
POSITION_OFFSET = 2          # T/opt/model.py:78 (position_offset=2), T/opt/model.py:232-244
MASK_FILL = -30000.0         # T/layers/attention.py:504-539 (masked scores are set to -30000)
DEFAULT_LN_EPS = 1e-5        # T/hlo.py:51 (batch_norm epsilon default), used by layer_norm T/hlo.py:84-105


def _f(t: torch.Tensor, dtype) -> torch.Tensor:
    return t.to(dtype)


def token_embedding(ids: torch.Tensor, embed_tokens: torch.Tensor) -> torch.Tensor:
    """x = embed_tokens.weight[input_ids]            (T/opt/model.py:163, T/hlo.py:1503-1533)"""
    return embed_tokens[ids.long()]


def learned_position_embedding(positions: torch.Tensor, embed_positions: torch.Tensor,
                               offset: int = POSITION_OFFSET) -> torch.Tensor:
    """p = embed_positions.weight[position_ids + 2]

    position_ids = max(cache_ids - start_ids, 0) (T/decoder.py:562-572); the table has
    max_position_embeddings + 2 rows (T/opt/gen_random_pretrained.py:51) and the offset of 2 is
    fixed in code (T/opt/model.py:232-244).  Without left padding position_ids = 0, 1, 2, ...
    """
    return embed_positions[positions.long() + offset]


def project(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """project_in / project_out: y = x @ W^T, no bias.

    The reference stores word_embed_proj_dim (T/opt/config.py:34) but never uses it, so there is no
    formula to cite.  Convention: project_in maps the token embedding [.., E] to [.., H] before the
    position embedding [.., H] is added; project_out maps the last hidden state (after the final
    LayerNorm when there is one) to [.., E] before the tied lm_head [V, E].
    """
    return x @ weight.t()


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               eps: float = DEFAULT_LN_EPS) -> torch.Tensor:
    """y = (x - mean) / sqrt(var + eps) * gamma + beta, statistics over the hidden axis, biased
    variance, all in 32-bit                                         (T/hlo.py:84-105, eps T/hlo.py:51).

    gamma/beta are optional: the reference always expects them (T/opt/model.py:98-99); the switch
    layer_norm_elementwise_affine=false (no gamma/beta) is this engine's convention.
    """
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """y = x @ W^T + b with W in the checkpoint's [out, in] orientation.

    q/k/v: T/opt/model.py:100-102 with T/hlo.py:398-399 (dot + bias); out_proj: T/opt/model.py:103,
    T/layers/attention.py:791-914; fc1/fc2: T/hlo.py:504-577.
    """
    y = x @ weight.t()
    if bias is not None:
        y = y + bias
    return y


def causal_mask(n_query: int, n_key: int, first_query_position: int = 0,
                window: Optional[int] = None) -> torch.Tensor:
    """mask[i, j] = (j <= position_i), position_i = first_query_position + i
    (T/hlo.py:941-1000: prefill uses 'LE' between key index and cache_ids, T/hlo.py:991-992).

    ``window`` (keys older than position_i - window + 1 are masked) is not an OPT feature; it is
    here so that kernels and toy parts can be tested at other settings than the engine's.
    """
    qpos = torch.arange(n_query) + first_query_position
    kpos = torch.arange(n_key)
    mask = kpos[None, :] <= qpos[:, None]
    if window is not None:
        mask &= kpos[None, :] > (qpos[:, None] - window)
    return mask


def attention_scores(q: torch.Tensor, k: torch.Tensor, head_dim: int,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Q = Q / sqrt(d) after the bias (T/opt/model.py:458-459, T/layers/attention.py:428-437);
    S = Q K^T per head (T/layers/attention.py:440-476).  q, k: [heads, T, d] -> [heads, Tq, Tk]."""
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    return (q * scale) @ k.transpose(-1, -2)


def masked_softmax(scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """S = where(mask, S, -30000); P = exp(S - max) / sum, in 32-bit
    (T/opt/model.py:508-516, T/layers/attention.py:504-539, T/hlo.py:880-904)."""
    s = torch.where(mask, scores, torch.full_like(scores, MASK_FILL))
    m = s.max(dim=-1, keepdim=True).values
    e = torch.exp(s - m)
    return e / e.sum(dim=-1, keepdim=True)


def attention_context(probs: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """C = P V per head (T/layers/attention.py:707-788).  [heads, Tq, Tk] x [heads, Tk, d]."""
    return probs @ v


def multi_head_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, n_heads: int,
                         n_kv_heads: Optional[int] = None, window: Optional[int] = None,
                         scale: Optional[float] = None) -> torch.Tensor:
    """The attention of one layer over a whole sequence h [T, H] (T/opt/model.py:388-524).

    Key/value heads equal heads for OPT (T/decoder.py:59); n_kv_heads < n_heads (each group of
    query heads reading one key/value head, T/layers/attention.py:455-460) is supported for tests of
    kernels at other settings.
    """
    T, H = h.shape
    n_kv_heads = n_kv_heads or n_heads
    q = linear(h, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias"))
    k = linear(h, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias"))
    v = linear(h, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias"))
    d = q.shape[-1] // n_heads
    q = q.view(T, n_heads, d).transpose(0, 1)
    k = k.view(T, n_kv_heads, d).transpose(0, 1)
    v = v.view(T, n_kv_heads, d).transpose(0, 1)
    if n_kv_heads != n_heads:
        rep = n_heads // n_kv_heads
        k = k.repeat_interleave(rep, dim=0)
        v = v.repeat_interleave(rep, dim=0)
    s = attention_scores(q, k, d, scale)
    p = masked_softmax(s, causal_mask(T, T, 0, window)[None])
    c = attention_context(p, v)                       # [heads, T, d]
    c = c.transpose(0, 1).reshape(T, n_heads * d)
    return linear(c, w[prefix + "out_proj.weight"], w.get(prefix + "out_proj.bias"))


def activation(name: str, x: torch.Tensor) -> torch.Tensor:
    """Activation looked up by config.activation_function (T/hlo.py:485-501): relu = max(x, 0)
    (T/activations.py:43-48); gelu_new = 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))
    (T/activations.py:20-41); sigmoid (T/activations.py:66-67); silu = x sigmoid(x)
    (T/activations.py:70-72); gelu is the exact form x Phi(x), which the reference does not have."""
    if name == "relu":
        return torch.clamp(x, min=0)
    if name == "gelu":
        return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))
    if name in ("gelu_new", "gelu_new_legacy"):
        return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))
    if name == "sigmoid":
        return 1.0 / (1.0 + torch.exp(-x))
    if name == "silu":
        return x / (1.0 + torch.exp(-x))
    raise ValueError(f"plain implementation has no activation {name!r}")


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, act: str) -> torch.Tensor:
    """a = act(h W1^T + b1); m = a W2^T + b2                        (T/hlo.py:504-577, :551-556)."""
    a = activation(act, linear(h, w[prefix + "fc1.weight"], w.get(prefix + "fc1.bias")))
    return linear(a, w[prefix + "fc2.weight"], w.get(prefix + "fc2.bias"))


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict) -> torch.Tensor:
    """One decoder layer over a whole sequence.

    Pre-LN (T/opt/model.py:336-376): h = LN1(x); x = x + Attn(h); h = LN2(x); x = x + FFN(h).
    Post-LN is rejected by the reference (T/opt/config.py:23-24); the convention here is
    x = LN1(x + Attn(x)); x = LN2(x + FFN(x)).
    """
    p = f"model.decoder.layers.{i}."
    eps = cfg.get("layer_norm_eps", DEFAULT_LN_EPS)
    heads = cfg["num_attention_heads"]
    act = cfg.get("activation_function", "relu")
    ln1 = (w.get(p + "self_attn_layer_norm.weight"), w.get(p + "self_attn_layer_norm.bias"))
    ln2 = (w.get(p + "final_layer_norm.weight"), w.get(p + "final_layer_norm.bias"))
    # Not a key of OPT's config.json: the reference takes a sliding window from NeuronConfig.sparse_attn
    # (T/opt/model.py:395-415; T/sparse_attn_utils.py:140-150: a row attends to itself and window_size before).
    window = cfg.get("sliding_window_size")
    window = None if window is None else window + 1
    if cfg.get("do_layer_norm_before", True):
        x = x + multi_head_attention(layer_norm(x, *ln1, eps), w, p + "self_attn.", heads, window=window)
        x = x + feed_forward(layer_norm(x, *ln2, eps), w, p, act)
    else:
        x = layer_norm(x + multi_head_attention(x, w, p + "self_attn.", heads, window=window), *ln1, eps)
        x = layer_norm(x + feed_forward(x, w, p, act), *ln2, eps)
    return x


def lm_head(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Final LayerNorm (pre-LN models only), optional project_out, logits = y @ lm_head^T without
    bias, in 32-bit (T/layers/transformer.py:148-213, T/opt/model.py:119-126,378-380).  lm_head is
    tied to embed_tokens when the checkpoint has no lm_head.weight (T/module.py:142-159)."""
    eps = cfg.get("layer_norm_eps", DEFAULT_LN_EPS)
    has_final_ln = cfg.get("do_layer_norm_before", True) and not cfg.get("_remove_final_layer_norm", False)
    if has_final_ln:
        x = layer_norm(x, w.get("model.decoder.final_layer_norm.weight"),
                       w.get("model.decoder.final_layer_norm.bias"), eps)
    if "model.decoder.project_out.weight" in w:
        x = project(x, w["model.decoder.project_out.weight"])
    head = w.get("lm_head.weight", w["model.decoder.embed_tokens.weight"])
    return x @ head.t()


def embed(ids: torch.Tensor, w: Dict[str, torch.Tensor], first_position: int = 0) -> torch.Tensor:
    """hidden = embed_tokens[ids] (projected in when E != H) + embed_positions[pos + 2]
    (T/opt/model.py:162-166)."""
    x = token_embedding(ids, w["model.decoder.embed_tokens.weight"])
    if "model.decoder.project_in.weight" in w:
        x = project(x, w["model.decoder.project_in.weight"])
    pos = torch.arange(ids.shape[0]) + first_position
    return x + learned_position_embedding(pos, w["model.decoder.embed_positions.weight"])


def forward_logits(ids, weights: Dict[str, torch.Tensor], cfg: dict,
                   dtype=torch.float32) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence of token ids (no padding)."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    w = {k: _f(v, dtype) for k, v in weights.items()}
    x = embed(ids, w)
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, i, cfg)
    return lm_head(x, w, cfg)


# ----------------------------------------------------------------------------------------------
# Sampling, as the reference's host loops do it.
# ----------------------------------------------------------------------------------------------

def greedy_token(logits: torch.Tensor) -> torch.Tensor:
    """argmax over the vocabulary (T/sampling.py:108-128); the lowest index wins a tie."""
    return torch.argmax(logits, dim=-1)


def filter_top_k_top_p(logits: torch.Tensor, top_k: Optional[int], top_p: Optional[float],
                       min_tokens_to_keep: int = 1) -> torch.Tensor:
    """Scores outside the top-k, or outside the smallest set of most likely tokens whose
    probability reaches top_p, become -inf (T/sampling.py:199-264)."""
    scores = logits.clone().float()
    if top_k is not None and top_k > 0:
        k = min(max(top_k, min_tokens_to_keep), scores.shape[-1])
        kth = torch.topk(scores, k, dim=-1).values[..., -1, None]
        scores = scores.masked_fill(scores < kth, -float("inf"))
    if top_p is not None and top_p < 1.0:
        sorted_scores, sorted_idx = torch.sort(scores, descending=True, dim=-1)
        cum = torch.softmax(sorted_scores, dim=-1).cumsum(dim=-1)
        remove = cum - torch.softmax(sorted_scores, dim=-1) >= top_p   # keep until the mass is reached
        remove[..., :min_tokens_to_keep] = False
        sorted_scores = sorted_scores.masked_fill(remove, -float("inf"))
        scores = torch.full_like(scores, -float("inf")).scatter(-1, sorted_idx, sorted_scores)
    return scores


def sampling_distribution(logits: torch.Tensor, temperature: float = 1.0,
                          top_k: Optional[int] = None, top_p: Optional[float] = None,
                          suppress: Optional[List[int]] = None) -> torch.Tensor:
    """Probabilities that the reference's loops draw from: logits / temperature, then the filters,
    then softmax in 32-bit (T/sampling.py:143-156 for top-k with the EOS score set to -inf,
    T/sampling.py:337-340 for temperature before top-p)."""
    scores = logits.float().clone()
    if suppress:
        scores[..., suppress] = -float("inf")
    scores = scores / temperature
    scores = filter_top_k_top_p(scores, top_k, top_p)
    return torch.softmax(scores, dim=-1)


def top_p_on_device(sorted_scores: torch.Tensor, top_p: float, top_p_min_tokens: int = 1) -> torch.Tensor:
    """The reference's on-device top-p over scores sorted from the largest down (T/hlo.py:2277-2364):
    p = softmax(scores); positions whose summed probability is still < top_p are counted; positions
    0 .. max(top_p_min_tokens - 1, that count) are kept.  Returns the mask of kept positions."""
    cum = torch.softmax(sorted_scores.double(), dim=-1).cumsum(dim=-1)      # 64-bit: the sums of a long row, exactly
    keep_positions = int((cum < top_p).sum())
    limit = max(top_p_min_tokens - 1, keep_positions)
    return torch.arange(sorted_scores.shape[-1]) <= limit


def multinomial_on_device(sorted_probs: torch.Tensor, uniform: float) -> int:
    """The reference's single draw over probabilities sorted from the largest down
    (T/hlo.py:2422-2467): the summed probabilities are divided by their last value and the answer
    is how many of them the uniform number exceeds (`deterministic`: the number is 0.5)."""
    cum = sorted_probs.double().cumsum(dim=-1)
    cum = cum / cum[-1]
    return int((uniform > cum).sum())


def sample_on_device(logits: torch.Tensor, top_k: Optional[int], top_p: float, top_p_min_tokens: int,
                     temperature: float, uniform: float = 0.5):
    """One row through the reference's on-device choice (T/layers/generation.py:147-199): scores /
    temperature, the top_k largest (sorted), top-p with its least number of tokens, softmax over
    what is left, one draw.  Returns (token, distance of the uniform number from the nearest
    summed probability), the latter so that a caller can tell a choice that rounding may flip."""
    scores = logits.float() / temperature
    k = scores.shape[-1] if not top_k else min(top_k, scores.shape[-1])
    vals, idx = torch.topk(scores, k)                      # sorted from the largest down
    if top_p < 1.0:
        keep = top_p_on_device(vals, top_p, top_p_min_tokens)
        vals, idx = vals[keep], idx[keep]
    probs = torch.softmax(vals.double(), dim=-1)
    j = multinomial_on_device(probs, uniform)
    cum = probs.cumsum(-1) / probs.sum()
    return int(idx[j]), float((cum - uniform).abs().min())


def greedy_generate(prompt: List[int], n_new: int, weights, cfg, dtype=torch.float32) -> List[int]:
    """Greedy continuation by running the whole sequence again for each new token."""
    ids = list(prompt)
    for _ in range(n_new):
        logits = forward_logits(ids, weights, cfg, dtype)
        ids.append(int(greedy_token(logits[-1])))
    return ids[len(prompt):]


# ----------------------------------------------------------------------------------------------
# The engine's own draw (no counterpart in the reference, whose host loops use torch's global
# generator, T/gpt_demo.py:101 and T/sampling.py:156): one uniform number per (seed, counter) from
# the Philox 4x32-10 counter generator, and the token whose interval of the summed probabilities,
# taken in index order, holds it.
# ----------------------------------------------------------------------------------------------

def philox_uniform(seed: int, counter: int) -> float:
    """First output word of Philox 4x32-10 with counter (counter, 0) and key = seed, as a number in
    [0, 1) with 32 bits."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [counter & mask, (counter >> 32) & mask, 0, 0]
    k = [seed & mask, (seed >> 32) & mask]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & mask, (p0 >> 32) ^ c[3] ^ k[1], p0 & mask]
        k = [(k[0] + W0) & mask, (k[1] + W1) & mask]
    return c[0] / 4294967296.0


def draw_in_index_order(probs: torch.Tensor, uniform: float):
    """The first token (in index order) at which the summed probability exceeds uniform * total.
    Returns (token, distance of uniform from the nearest summed probability)."""
    cum = probs.double().cumsum(-1)
    cum = cum / cum[-1]
    tok = int((cum <= uniform).sum())
    tok = min(tok, probs.shape[-1] - 1)
    return tok, float((cum - uniform).abs().min())
