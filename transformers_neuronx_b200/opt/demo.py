"""opt_demo: the reference's command line (src/transformers_neuronx/gpt_demo.py:31-150,
opt/demo.py:19-29) for this engine.

    opt_demo [--amp f32|f16|bf16] save <folder> --random --config cfg.json [--seed N]
    opt_demo [--amp f32|f16|bf16] [--model_name <folder>] save <folder>         (re-save a local checkpoint)
    opt_demo [--amp f32|f16|bf16] run <folder> [--batch_size 4] [--n_positions 128] [--print_latency]
             [--top_k 50] [--temperature 1.0] [--top_p 1.0] [--prompt_ids 2,100,200]
             [--sparse_attn window --window_size 128]

`save` casts attention, fc1, fc2 and embedding matrices to --amp and keeps LayerNorm tensors in
32-bit, as the reference's amp_callback does (opt/demo.py:23-29).  `run` seeds with 15213, repeats
one prompt batch_size times and samples to n_positions (gpt_demo.py:100-150).  With tokenizer files
in the folder and the `transformers` tokenizer classes importable the prompt is the reference's
"Hello, I'm a language model,"; otherwise token ids go in and out.  Options of the reference that
only mean something on Neuron hardware (--tp_degree, --unroll, --quantize, the block-sparse numbers ...) are
accepted and ignored.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch

from ..config import config_from_dict, load_config
from ..models.decoder import DecoderModel
from ..weights import load_tensors, save_safetensors, write_model_folder
from .model import OPTForSampling

PROMPT_TEXT = "Hello, I'm a language model,"


def _parser():
    ap = argparse.ArgumentParser(prog="opt_demo")
    ap.add_argument("--amp", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--model_name", default=None, help="local folder of a pretrained model (for save)")
    sub = ap.add_subparsers(dest="which", required=True)
    sp = sub.add_parser("save")
    sp.add_argument("save", help="Directory to save the model")
    sp.add_argument("--random", action="store_true", help="random weights from --config")
    sp.add_argument("--config", type=str, default="", help="path/to/config.json")
    sp.add_argument("--seed", type=int, default=0)
    rp = sub.add_parser("run")
    rp.add_argument("load")
    rp.add_argument("--batch_size", type=int, default=4, help="Input batch size")
    rp.add_argument("--n_positions", type=int, default=128, help="Input sequence length")
    rp.add_argument("--print_latency", action="store_true", help="Print latency of each step")
    rp.add_argument("--top_k", type=int, default=50)
    rp.add_argument("--temperature", type=float, default=1.0)
    rp.add_argument("--top_p", type=float, default=1.0)
    rp.add_argument("--prompt_ids", type=str, default=None, help="comma-separated token ids of the prompt")
    rp.add_argument("--sparse_attn", type=str, default=None, choices=[None, "blk_sparse", "custom", "window"],
                    help="'window': sliding-window attention (the other patterns are not built)")
    rp.add_argument("--window_size", type=int, default=128, help="Window size for sliding-window attention.")
    for name in ("--tp_degree", "--unroll", "--context_length_estimate", "--blk_size",
                 "--num_global_blks", "--num_local_blks", "--num_random_blks"):
        rp.add_argument(name, type=int, default=None, help=argparse.SUPPRESS)
    rp.add_argument("--quantize", action="store_true", help=argparse.SUPPRESS)
    return ap


def save(args):
    dtype = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[args.amp]
    if args.random:
        assert args.config, "Please provide the config.json like: --config=./config.json"
        assert os.path.exists(args.config), f"File {args.config} does not exist."
        with open(args.config) as fp:
            arch, cfg = config_from_dict(json.load(fp))
        specs = DecoderModel(arch.build_spec(cfg)).tensor_specs()
        write_model_folder(args.save, cfg, specs, args.seed, matrix_dtype=dtype)
    else:
        src = args.model_name
        if not src or not os.path.isdir(src):
            raise SystemExit("save without --random needs --model_name <local folder>; a model cannot be "
                             "fetched by name without a network")
        arch, cfg = load_config(src)
        specs = DecoderModel(arch.build_spec(cfg)).tensor_specs()
        tensors = load_tensors(src, specs)
        out = {}
        for s in specs:
            if s.tied_to is not None and tensors[s.name] is tensors.get(s.tied_to):
                continue
            t = tensors[s.name]
            out[s.name] = t.to(torch.float32) if s.kind.startswith("norm") else t.to(dtype)
        cfg.save(args.save)
        save_safetensors(out, os.path.join(args.save, "model.safetensors"), metadata={"format": "pt"})
    print(f"saved {args.save}")


def _tokenizer(folder):
    if not any(os.path.exists(os.path.join(folder, f)) for f in ("tokenizer.json", "vocab.json")):
        return None
    try:
        from transformers import AutoTokenizer      # a tokenizer, not model code
        return AutoTokenizer.from_pretrained(folder)
    except Exception:
        return None


def run(args):
    torch.manual_seed(15213)
    print("running OPTForSampling.from_pretrained")
    neuron_config = None
    if args.sparse_attn:                                    # gpt_demo.py:107-123
        if args.sparse_attn != "window":
            raise NotImplementedError("Interface for other attention patterns not implemented yet!")
        from ..config import NeuronConfig, SlidingWindowAttnConfig, SparseAttnConfig
        neuron_config = NeuronConfig(sparse_attn=SparseAttnConfig(
            attn_type="window", causal=True, sparse_attn_config=SlidingWindowAttnConfig(window_size=args.window_size)))
    model = OPTForSampling.from_pretrained(args.load, batch_size=args.batch_size, amp=args.amp,
                                           n_positions=args.n_positions, neuron_config=neuron_config)
    print("running model.to_neuron")
    model.to_neuron()
    tok = _tokenizer(args.load)
    if args.prompt_ids:
        ids = [int(t) for t in args.prompt_ids.split(",")]
    elif tok is not None:
        ids = tok.encode(PROMPT_TEXT)
    else:
        v = model.config.vocab_size
        ids = [model.config.bos_token_id] + [3 + (7 * i) % (v - 3) for i in range(1, 9)]
    input_ids = torch.as_tensor([ids] * args.batch_size)
    if args.print_latency:
        runner = model.engine.runner
        inner = runner.step

        def timed(entries, *args, **kwargs):
            torch.cuda.synchronize()
            t0 = time.time()
            out = inner(entries, *args, **kwargs)
            torch.cuda.synchronize()
            print(f"cache_offset: {max(runner.cache.length(e.rid) for e in entries) - 1}")
            print(f"Latency: {math.ceil((time.time() - t0) * 1000)} ms")
            return out
        runner.step = timed
    print("running model.sample")
    seq = model.sample(input_ids, sequence_length=args.n_positions, top_k=args.top_k,
                       temperature=args.temperature, top_p=args.top_p, seed=15213)
    print("generated_sequence=", seq)
    if tok is not None:
        print([tok.decode(s) for s in seq])
    return seq


def main(argv=None):
    args = _parser().parse_args(argv)
    if args.which == "save":
        save(args)
    else:
        run(args)


if __name__ == "__main__":
    main()
