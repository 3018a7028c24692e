"""Runs the reference's own OPT layer code on the CPU and writes the logits as a golden file.

The reference's decoder exists only as Python that builds an HLO graph for the Neuron compiler
(src/transformers_neuronx/opt/model.py:272-524 calls layers/attention.py, layers/transformer.py and
hlo.py, which call methods of a `scribe` object of torch_neuronx.pyhlo).  That Python is ordinary
code: every operation is a call `dtype[sizes].Op(operands, attributes)`.  Here the scribe is
replaced by a stand-in whose operations are evaluated at once with torch on the CPU (each one
checked against the shape the reference declares for it), so the reference's own functions compute
numbers: the mask conventions, the order of bias, scale and casts, the split softmax of a decode
step, the cache update, LayerNorm and the head are the reference's, not a restatement.

    python tests/golden/reference_graph_eager.py /path/to/transformers-neuronx/src

writes opt_reference_logits.json beside this script: the 32-bit logits of a tiny OPT (pre-norm,
biases, affine norms: what the reference supports) for a left-padded batch of two prompts at every
prompt position, and for three decode steps after them.  The weights are closed-form functions of
their indices (golden_weights below), so the test that compares the plain implementation with the
file needs nothing but this module's formulas.  The Neuron SDK modules that the reference imports at
module level are replaced by empty stand-ins; nothing of them is called.
"""
import json
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CONFIG = dict(vocab_size=96, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, ffn_dim=64,
              max_position_embeddings=30, word_embed_proj_dim=32, do_layer_norm_before=True, enable_bias=True,
              layer_norm_elementwise_affine=True, activation_function="relu", eos_token_id=2, pad_token_id=1,
              torch_dtype="float32")
PROMPT_LEN, N_DECODE, N_POSITIONS = 10, 3, 16
START_IDS = [0, 3]                    # row 1 is left-padded by three places


def golden_weights(cfg=CONFIG):
    """{HF tensor name: 32-bit tensor}: every value a closed-form function of its index."""
    H, F, V, P = cfg["hidden_size"], cfg["ffn_dim"], cfg["vocab_size"], cfg["max_position_embeddings"] + 2
    k = [0]

    def wave(*shape, scale=0.2, shift=0.0):
        k[0] += 1
        n = math.prod(shape)
        i = torch.arange(n, dtype=torch.float64)
        return (shift + scale * torch.sin(i * (0.37 + 0.011 * k[0]) + 1.3 * k[0])).to(torch.float32).view(*shape)

    w = {"model.decoder.embed_tokens.weight": wave(V, H, scale=0.5),
         "model.decoder.embed_positions.weight": wave(P, H, scale=0.3),
         "model.decoder.final_layer_norm.weight": wave(H, scale=0.2, shift=1.0),
         "model.decoder.final_layer_norm.bias": wave(H, scale=0.1)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.decoder.layers.{i}."
        for n in ("q", "k", "v", "out"):
            w[p + f"self_attn.{n}_proj.weight"] = wave(H, H, scale=0.25)
            w[p + f"self_attn.{n}_proj.bias"] = wave(H, scale=0.1)
        w[p + "self_attn_layer_norm.weight"] = wave(H, scale=0.2, shift=1.0)
        w[p + "self_attn_layer_norm.bias"] = wave(H, scale=0.1)
        w[p + "fc1.weight"] = wave(F, H, scale=0.25)
        w[p + "fc1.bias"] = wave(F, scale=0.1)
        w[p + "fc2.weight"] = wave(H, F, scale=0.2)
        w[p + "fc2.bias"] = wave(H, scale=0.1)
        w[p + "final_layer_norm.weight"] = wave(H, scale=0.2, shift=1.0)
        w[p + "final_layer_norm.bias"] = wave(H, scale=0.1)
    return w


def golden_tokens(cfg=CONFIG):
    """[2, PROMPT_LEN + N_DECODE] token ids; row 1 starts with START_IDS[1] pad tokens."""
    V = cfg["vocab_size"]
    rows = [[3 + (7 * i + 11 * b * b + 5) % (V - 3) for i in range(PROMPT_LEN + N_DECODE)] for b in range(2)]
    for b, s in enumerate(START_IDS):
        rows[b][:s] = [cfg["pad_token_id"]] * s
    return rows


# ---- the eager stand-in for torch_neuronx.pyhlo's scribe ------------------------------------------
_TORCH = {"f32": torch.float32, "f64": torch.float64, "f16": torch.float16, "bf16": torch.bfloat16,
          "s64": torch.int64, "s32": torch.int32, "s16": torch.int16, "s8": torch.int8,
          "u64": torch.int64, "u32": torch.int64, "u16": torch.int32, "u8": torch.uint8, "pred": torch.bool}


class Value:
    """What an operation returns: the numbers, and the .sizes / .dtype / .scribe the reference's code reads."""

    def __init__(self, data, dtype):
        self.data, self.dtype, self.scribe = data, dtype, dtype.scribe
        self.sizes = tuple(data.shape)

    def __repr__(self):
        return f"Value({self.dtype.name}{list(self.sizes)})"


class TupleValue:
    def __init__(self, values, scribe):
        self.values, self.scribe = list(values), scribe

    def get_tuple_element(self, i):          # pyhlo: the element's shape; the value itself serves
        return self.values[i]


class Shape:
    """dtype[sizes]: calling .Op(...) on it evaluates the operation and checks the declared shape."""

    def __init__(self, dtype, sizes):
        self.dtype, self.sizes, self.scribe = dtype, tuple(int(s) for s in sizes), dtype.scribe

    def __getattr__(self, op):
        if op.startswith("_"):
            raise AttributeError(op)
        fn = _OPS.get(op)
        if fn is None:
            raise NotImplementedError(f"HLO operation {op} is not evaluated by this stand-in")

        def call(*operands, **attrs):
            out = fn(self, *operands, **attrs)
            if isinstance(out, torch.Tensor):
                want = _TORCH[self.dtype.name]
                assert tuple(out.shape) == self.sizes, f"{op}: result {tuple(out.shape)}, declared {self.sizes}"
                return Value(out.to(want), self.dtype)
            return out
        return call


class DType:
    def __init__(self, scribe, name):
        self.scribe, self.name = scribe, name
        self.dtype = self               # hlo.py writes u32.dtype[sizes] in places

    def __getitem__(self, sizes):
        if not isinstance(sizes, (tuple, list)):
            sizes = (sizes,)
        return Shape(self, sizes)

    def __getattr__(self, op):          # dtype.Constant(...): an operation on a scalar shape
        if op.startswith("_"):
            raise AttributeError(op)
        return getattr(Shape(self, ()), op)

    def __repr__(self):
        return f"<{self.name}>"


class TupleShape:
    def __init__(self, scribe, shapes):
        self.scribe, self.shapes = scribe, shapes

    def __getattr__(self, op):
        if op.startswith("_"):
            raise AttributeError(op)
        fn = _TUPLE_OPS.get(op)
        if fn is None:
            raise NotImplementedError(f"tuple-shaped HLO operation {op} is not evaluated by this stand-in")
        return lambda *operands, **attrs: fn(self, *operands, **attrs)


class Scribe:
    def __init__(self):
        for name in _TORCH:
            setattr(self, name, DType(self, name))

    def tuple(self, *shapes):
        return TupleShape(self, shapes)


def _d(v):
    return v.data


def _binary(fn):
    return lambda shape, a, b: fn(_d(a), _d(b))


def _compare(shape, a, b, comparison_direction):
    x, y = _d(a), _d(b)
    return {"LT": x < y, "LE": x <= y, "GT": x > y, "GE": x >= y, "EQ": x == y, "NE": x != y}[comparison_direction]


def _broadcast(shape, x, dimensions):
    """Operand dimension i becomes result dimension dimensions[i]; the others are repeated."""
    t = _d(x)
    view = [1] * len(shape.sizes)
    for i, dim in enumerate(dimensions):
        view[dim] = t.shape[i]
    return t.reshape(view).expand(shape.sizes).clone()


def _dot(shape, lhs, rhs, dot_dimension_numbers):
    a, b = _d(lhs), _d(rhs)
    dn = dot_dimension_numbers
    lb, rb = list(dn.get("lhs_batch_dimensions", [])), list(dn.get("rhs_batch_dimensions", []))
    lc, rc = list(dn["lhs_contracting_dimensions"]), list(dn["rhs_contracting_dimensions"])
    lf = [i for i in range(a.dim()) if i not in lb + lc]
    rf = [i for i in range(b.dim()) if i not in rb + rc]
    letters = "abcdefghijklmnopqrstuvwxyz"
    la, lbn, nxt = [None] * a.dim(), [None] * b.dim(), 0
    for i, j in zip(lb, rb):
        la[i] = lbn[j] = letters[nxt]; nxt += 1
    for i, j in zip(lc, rc):
        la[i] = lbn[j] = letters[nxt]; nxt += 1
    for i in lf:
        la[i] = letters[nxt]; nxt += 1
    for j in rf:
        lbn[j] = letters[nxt]; nxt += 1
    out = [la[i] for i in lb] + [la[i] for i in lf] + [lbn[j] for j in rf]     # XLA: batch, lhs free, rhs free
    wide = torch.float64 if a.dtype.is_floating_point else a.dtype
    return torch.einsum(f"{''.join(la)},{''.join(lbn)}->{''.join(out)}", a.to(wide), b.to(wide)).to(a.dtype)


def _probe_reduction(to_apply, dtype):
    """Which reduction a sub-computation is: it is evaluated on the scalars 2 and 3."""
    s = dtype.scribe
    params = iter([Value(torch.tensor(2, dtype=_TORCH[dtype.name]), dtype), Value(torch.tensor(3, dtype=_TORCH[dtype.name]), dtype)])
    saved = _OPS["Parameter"]
    _OPS["Parameter"] = lambda shape, parameter_number=None: next(params).data
    try:
        r = float(to_apply(s).data)
    finally:
        _OPS["Parameter"] = saved
    return {5.0: "sum", 3.0: "max", 2.0: "min", 6.0: "prod"}[r]


def _reduce(shape, x, init, dimensions, to_apply):
    t, kind = _d(x), _probe_reduction(to_apply, x.dtype)
    dims = tuple(dimensions)
    if kind == "sum":
        wide = t.to(torch.float64) if t.dtype.is_floating_point else t
        return (wide.sum(dims) + _d(init).to(wide.dtype)).to(t.dtype)
    if kind == "max":
        return torch.maximum(t.amax(dims), _d(init))
    if kind == "min":
        return torch.minimum(t.amin(dims), _d(init))
    raise NotImplementedError(kind)


def _constant(shape, constant_value):
    return torch.tensor(constant_value, dtype=_TORCH[shape.dtype.name]).reshape(shape.sizes) if shape.sizes == () \
        else torch.full(shape.sizes, constant_value, dtype=_TORCH[shape.dtype.name])


def _iota(shape, dimensions):
    (dim,) = dimensions
    view = [1] * len(shape.sizes)
    view[dim] = shape.sizes[dim]
    return torch.arange(shape.sizes[dim]).reshape(view).expand(shape.sizes).clone()


def _slice(shape, x, slice_dimensions):
    t = _d(x)
    idx = tuple(slice(d["start"], d["limit"], d.get("stride", 1)) for d in slice_dimensions)
    return t[idx].clone()


def _dynamic_slice(shape, x, *starts, dynamic_slice_sizes):
    t = _d(x)
    idx = []
    for dim, (s, n) in enumerate(zip(starts, dynamic_slice_sizes)):
        b = int(_d(s).reshape(-1)[0])
        b = max(0, min(b, t.shape[dim] - n))                   # XLA clamps the start
        idx.append(slice(b, b + n))
    return t[tuple(idx)].clone()


def _dynamic_update_slice(shape, x, update, *starts):
    t = _d(x).clone()
    u = _d(update)
    idx = []
    for dim, s in enumerate(starts):
        b = int(_d(s).reshape(-1)[0])
        b = max(0, min(b, t.shape[dim] - u.shape[dim]))
        idx.append(slice(b, b + u.shape[dim]))
    t[tuple(idx)] = u
    return t


def _gather(shape, operand, indices, gather_dimension_numbers, gather_slice_sizes, **_):
    """The one form the OPT path uses: rows of a table picked by an index vector."""
    t, ix = _d(operand), _d(indices).long()
    dn = gather_dimension_numbers
    if list(dn.get("collapsed_slice_dims", [])) == [0] and list(dn.get("start_index_map", [])) == [0] and \
            list(gather_slice_sizes) == [1] + list(t.shape[1:]):
        return t[ix.reshape(-1)].reshape(shape.sizes)
    raise NotImplementedError(f"Gather with {dn}")


def _scatter(shape, operand, indices, updates, scatter_dimension_numbers, to_apply=None, **_):
    """The cache update: rows (first dimension) of `operand` named by `indices` are replaced (the
    sub-computation is the reference's assign function: the update wins)."""
    t, ix, u = _d(operand).clone(), _d(indices).long().reshape(-1), _d(updates)
    dn = scatter_dimension_numbers
    if list(dn.get("scatter_dims_to_operand_dims", [])) == [0] and list(dn.get("inserted_window_dims", [])) == [0]:
        t[ix] = u.reshape(len(ix), *t.shape[1:])
        return t
    raise NotImplementedError(f"Scatter with {dn}")


def _custom_call(shape, *operands, custom_call_target, backend_config=None, **_):
    if custom_call_target == "AwsNeuronSoftmax":
        dim = int(backend_config.decode() if isinstance(backend_config, bytes) else backend_config)
        return torch.softmax(_d(operands[0]).to(torch.float64), dim=dim).to(_d(operands[0]).dtype)
    raise NotImplementedError(f"custom call {custom_call_target}")


def _batch_norm_training(tshape, x, scale, offset, epsilon, feature_index):
    """XLA BatchNormTraining: statistics over every dimension but feature_index (biased variance)."""
    t = _d(x).to(torch.float64)
    dims = tuple(i for i in range(t.dim()) if i != feature_index)
    mean = t.mean(dims, keepdim=True)
    var = ((t - mean) ** 2).mean(dims, keepdim=True)
    view = [1] * t.dim(); view[feature_index] = -1
    y = (t - mean) / torch.sqrt(var + epsilon) * _d(scale).to(torch.float64).view(view) + _d(offset).to(torch.float64).view(view)
    dt = x.dtype
    return TupleValue([Value(y.to(_d(x).dtype), dt), Value(mean.reshape(-1).to(_d(x).dtype), dt),
                       Value(var.reshape(-1).to(_d(x).dtype), dt)], tshape.scribe)


_OPS = {
    "Parameter": None,
    "Constant": _constant,
    "Iota": _iota,
    "Broadcast": _broadcast,
    "Reshape": lambda shape, x: _d(x).reshape(shape.sizes).clone(),
    "Transpose": lambda shape, x, dimensions: _d(x).permute(*dimensions).contiguous(),
    "Convert": lambda shape, x: _d(x).to(_TORCH[shape.dtype.name]),
    "Add": _binary(torch.add), "Subtract": _binary(torch.sub), "Multiply": _binary(torch.mul),
    "Divide": lambda shape, a, b: (_d(a) / _d(b)) if _d(a).dtype.is_floating_point else torch.div(_d(a), _d(b), rounding_mode="trunc"),
    "Maximum": _binary(torch.maximum), "Minimum": _binary(torch.minimum),
    "And": _binary(torch.logical_and), "Or": _binary(torch.logical_or), "Not": lambda shape, a: ~_d(a),
    "Exp": lambda shape, a: torch.exp(_d(a)), "Sqrt": lambda shape, a: torch.sqrt(_d(a)),
    "Rsqrt": lambda shape, a: torch.rsqrt(_d(a)), "Tanh": lambda shape, a: torch.tanh(_d(a)),
    "Log": lambda shape, a: torch.log(_d(a)), "Logistic": lambda shape, a: torch.sigmoid(_d(a)),
    "Compare": _compare,
    "Select": lambda shape, pred, a, b: torch.where(_d(pred), _d(a), _d(b)),
    "Dot": _dot,
    "Reduce": _reduce,
    "Slice": _slice,
    "DynamicSlice": _dynamic_slice,
    "DynamicUpdateSlice": _dynamic_update_slice,
    "Concatenate": lambda shape, *xs, dimensions: torch.cat([_d(x) for x in xs], dim=dimensions[0]),
    "Gather": _gather,
    "Scatter": _scatter,
    "CustomCall": _custom_call,
    "GetTupleElement": lambda shape, tup, tuple_index: tup.values[tuple_index].data,
}
_TUPLE_OPS = {"BatchNormTraining": _batch_norm_training}


def value(scribe, tensor, name):
    return Value(tensor.to(_TORCH[name]), getattr(scribe, name))


# ---- the driver ------------------------------------------------------------------------------------
def run_reference(src):
    sys.path.insert(0, HERE)
    from make_reference_goldens import stub_neuron_sdk
    sys.path.insert(0, src)
    stub_neuron_sdk()
    from transformers_neuronx.config import NeuronConfig
    from transformers_neuronx.opt.model import OPTForSamplingNoEmbeddingHlo

    cfg = CONFIG
    H, nh, L = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_hidden_layers"]
    d = H // nh
    w = golden_weights()
    toks = torch.tensor(golden_tokens())
    B = toks.shape[0]
    s = Scribe()
    builder = OPTForSamplingNoEmbeddingHlo(1, H, cfg["activation_function"], eos_token_id=cfg["eos_token_id"], amp="f32",
                                           neuron_config=NeuronConfig(), position_offset=2)
    v = lambda t, name="f32": value(s, t, name)
    dec = "model.decoder."

    def layer_weights(i):
        """In the orientation the reference's loader gives the graph (opt/model.py:94-130): q, k, v and
        fc1 transposed to [in, out], out_proj and fc2 as stored."""
        p = f"{dec}layers.{i}."
        g = lambda n: w[p + n]
        return dict(
            pre_attn_ln_weight=v(g("self_attn_layer_norm.weight")), pre_attn_ln_bias=v(g("self_attn_layer_norm.bias")),
            attn_q_weight=v(g("self_attn.q_proj.weight").t().contiguous()), attn_q_scales=None, attn_q_bias=v(g("self_attn.q_proj.bias")),
            attn_k_weight=v(g("self_attn.k_proj.weight").t().contiguous()), attn_k_scales=None, attn_k_bias=v(g("self_attn.k_proj.bias")),
            attn_v_weight=v(g("self_attn.v_proj.weight").t().contiguous()), attn_v_scales=None, attn_v_bias=v(g("self_attn.v_proj.bias")),
            attn_out_weight=v(g("self_attn.out_proj.weight")), attn_out_scales=None, attn_out_bias=v(g("self_attn.out_proj.bias")),
            post_attn_ln_weight=None, post_attn_ln_bias=None,
            pre_mlp_ln_weight=v(g("final_layer_norm.weight")), pre_mlp_ln_bias=v(g("final_layer_norm.bias")),
            mlp_in_weight=v(g("fc1.weight").t().contiguous()), mlp_in_scales=None, mlp_in_bias=v(g("fc1.bias")),
            mlp_out_weight=v(g("fc2.weight")), mlp_out_scales=None, mlp_out_bias=v(g("fc2.bias")),
            post_mlp_ln_weight=None, post_mlp_ln_bias=None)

    wte, wpe = v(w[dec + "embed_tokens.weight"]), v(w[dec + "embed_positions.weight"])
    ln_f = (v(w[dec + "final_layer_norm.weight"]), v(w[dec + "final_layer_norm.bias"]))
    lm_head = v(w[dec + "embed_tokens.weight"].t().contiguous())      # tied; [H, V] as the graph takes it
    start_ids = v(torch.tensor(START_IDS), "s32")

    def step(input_ids, cache_ids, n_positions, caches):
        """One call of the reference's graph: embedding, pre_layer (masks), the layers, the head with
        all positions' logits.  caches: per layer (K, V) Values or None (prefill)."""
        builder.n_positions = n_positions
        T = input_ids.shape[1]
        last = v(torch.tensor([T - 1]), "s32")
        cid = v(cache_ids, "s32")
        hidden = builder.embedding(v(input_ids, "s32"), cid, start_ids, last, None, None, None, wte, wpe)
        hidden, last_token_id, cws, cid2, sid, mask, active_mask = builder.pre_layer(
            hidden, cid, start_ids, last, None, None, v(torch.tensor([0]), "s32"))
        out_caches = []
        for i in range(L):
            if caches is None:
                kc = vc = v(torch.zeros(n_positions, B, nh, d))
            else:
                kc, vc = caches[i]
            hidden, kc, vc = builder.layer(hidden, last_token_id, cws, cid2, sid, mask, active_mask, kc, vc, **layer_weights(i))
            out_caches.append((kc, vc))
        logits = builder.ln_lm_head(hidden, last_token_id, ln_f[0], ln_f[1], lm_head, None, return_all_outputs=True)
        return logits.data.permute(2, 1, 0).contiguous(), out_caches       # [V, T, B] -> [B, T, V]

    T0 = PROMPT_LEN
    prefill_logits, caches = step(toks[:, :T0], torch.arange(T0), T0, None)
    # the prompt's keys and values go into a cache of N_POSITIONS rows, as the reference's decoder does
    full = []
    for kc, vc in caches:
        K, V_ = torch.zeros(N_POSITIONS, B, nh, d), torch.zeros(N_POSITIONS, B, nh, d)
        K[:T0], V_[:T0] = kc.data, vc.data
        full.append((v(K), v(V_)))
    decode_logits = []
    for t in range(T0, T0 + N_DECODE):
        lg, full = step(toks[:, t:t + 1], torch.tensor([t]), N_POSITIONS, full)
        decode_logits.append(lg[:, 0])
    return prefill_logits, torch.stack(decode_logits, dim=1)


def main(src):
    prefill, decode = run_reference(src)
    out = {"config": CONFIG, "start_ids": START_IDS, "tokens": golden_tokens(),
           "prefill_logits": [[[round(float(x), 7) for x in row] for row in b] for b in prefill],
           "decode_logits": [[[round(float(x), 7) for x in row] for row in b] for b in decode]}
    with open(os.path.join(HERE, "opt_reference_logits.json"), "w") as fp:
        json.dump(out, fp)
    print("wrote opt_reference_logits.json", tuple(prefill.shape), tuple(decode.shape))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.environ.get("TNX_REFERENCE", "reference"), "src"))
