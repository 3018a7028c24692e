"""opt_gen_random_pretrained <config.json> <folder> [--seed N]: a model folder with random weights.

Same two positional arguments as src/transformers_neuronx/opt/gen_random_pretrained.py:23-29; the
folder holds config.json and model.safetensors instead of a split checkpoint, and every tensor is
random (see weights/random_init.py)."""
from __future__ import annotations

import argparse
import json

from ..config import config_from_dict
from ..models.decoder import DecoderModel
from ..weights import write_model_folder


def gen_random_pretrained(config_path: str, save: str, seed: int = 0):
    with open(config_path) as fp:
        arch, cfg = config_from_dict(json.load(fp))      # the model class is chosen by config.json
    specs = DecoderModel(arch.build_spec(cfg)).tensor_specs()
    write_model_folder(save, cfg, specs, seed)
    return cfg


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("name", help="path to an OPT config.json")
    ap.add_argument("save", help="target folder to save the model")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    gen_random_pretrained(a.name, a.save, a.seed)
    print(f"done saving {a.save}")


if __name__ == "__main__":
    main()
