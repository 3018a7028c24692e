"""Makes the golden files of this folder from aws-neuron/transformers-neuronx's own code, run on the CPU.

What of the reference can run here: its random-checkpoint writer (tensor names and shapes of an OPT
checkpoint) and its host-side sampling filter (top-k / top-p).  Its model code cannot: the decoder
exists only as an HLO graph for the Neuron compiler.  The Neuron SDK packages that the reference
imports at module level (torch_neuronx, libneuronxla, neuronxcc) are replaced by empty stand-ins;
nothing of them is called.

    python tests/golden/make_reference_goldens.py /path/to/transformers-neuronx/src

writes opt_tensor_names.json and top_k_top_p.json beside this script.
"""
import json
import os
import sys
import tempfile
import types
from unittest import mock

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CONFIG = dict(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, ffn_dim=256,
              max_position_embeddings=128, word_embed_proj_dim=64, do_layer_norm_before=True, init_std=0.02,
              torch_dtype="float32", activation_function="relu", eos_token_id=2, pad_token_id=1)


class _Stub(types.ModuleType):
    """An empty stand-in for a Neuron SDK module: any attribute is a mock, any submodule another stub."""
    __version__ = "0.0"
    __path__ = []

    def __getattr__(self, key):
        if key.startswith("__"):
            raise AttributeError(key)
        return mock.MagicMock(name=f"{self.__name__}.{key}")


class _StubFinder:
    PREFIXES = ("torch_neuronx", "libneuronxla", "neuronxcc")

    def find_spec(self, name, path=None, target=None):
        import importlib.machinery
        if name.split(".")[0] in self.PREFIXES:
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        return _Stub(spec.name)

    def exec_module(self, module):
        pass


def stub_neuron_sdk():
    sys.meta_path.insert(0, _StubFinder())


def main(src):
    sys.path.insert(0, src)
    stub_neuron_sdk()
    from transformers_neuronx.opt import gen_random_pretrained as gen
    from transformers_neuronx import sampling

    with tempfile.TemporaryDirectory() as tmp:
        cfg_path = os.path.join(tmp, "config.json")
        with open(cfg_path, "w") as fp:
            json.dump(CONFIG, fp)
        out = os.path.join(tmp, "model")
        gen.gen_random_pretrained(cfg_path, out)
        with open(os.path.join(out, "pytorch_model.bin", "key_to_filename.json")) as fp:
            key_to_file = json.load(fp)
        names = {}
        for key, fname in key_to_file.items():
            t = torch.load(os.path.join(out, "pytorch_model.bin", fname))
            names[key] = list(t.shape)
    with open(os.path.join(HERE, "opt_tensor_names.json"), "w") as fp:
        json.dump({"config": CONFIG, "tensors": names}, fp, indent=1, sort_keys=True)

    g = torch.Generator().manual_seed(0)
    cases = []
    for top_k, top_p in ((5, None), (None, 0.7), (12, 0.6), (50, 0.95), (None, 0.2), (1, None)):
        scores = (torch.randn(3, 97, generator=g) * 2.0)
        vals, idx = sampling.top_k_top_p_filtering(scores.clone(), top_k=top_k, top_p=top_p)
        kept = [sorted(int(i) for i, v in zip(idx[b].tolist(), vals[b].tolist()) if v != -float("inf")) for b in range(3)]
        cases.append({"top_k": top_k, "top_p": top_p, "scores": scores.tolist(), "kept": kept})
    with open(os.path.join(HERE, "top_k_top_p.json"), "w") as fp:
        json.dump(cases, fp)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.environ.get("TNX_REFERENCE", "reference"), "src"))
