"""From a model folder (config.json, model.safetensors) to a model on the GPU."""
from __future__ import annotations

import sys
import time
import warnings

import torch

from ..config import canonical_dtype, load_config
from ..kernels import build as kbuild
from ..models.decoder import DecoderModel
from ..parts.base import rounding_report
from ..weights import load_tensors

_TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def require_cuda(device="cuda:0") -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on a GPU only (sm_100a); there is no CPU path")
    dev = torch.device(device)
    major, minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"the kernels are built for sm_100a (B200); device {dev} is sm_{major}{minor}")
    return dev


def build_model(spec, tensors, dtype: str, device="cuda:0", verbose=True) -> DecoderModel:
    """A ModelSpec and its {name: tensor} -> a DecoderModel on the device, kernels compiled."""
    dev = require_cuda(device)
    torch.cuda.set_device(dev)
    model = DecoderModel(spec)
    act = _TORCH_DTYPE[canonical_dtype(dtype)]
    # the libraries' flavour: the engine's 16-bit type, or (32-bit engine) that of the stored matrices
    sixteen = act if act != torch.float32 else (
        torch.float16 if any(t.dtype == torch.float16 for t in tensors.values()) else torch.bfloat16)
    kbuild.build_many(kbuild.with_flavour(model.libraries(act), sixteen), verbose=verbose)
    rounding_report()
    model.load(tensors, dev, act)
    n, example = rounding_report()
    if n:
        warnings.warn(f"{n} tensors are stored in another 16-bit type than the engine's and were rounded to "
                      f"{canonical_dtype(dtype)} (e.g. {example}): the logits are no longer the checkpoint's own; "
                      f"run the engine in the checkpoint's type, or in float32, to avoid this")
    return model


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0", verbose=True, spec_hook=None):
    """Returns (model, typed config).  The model class is chosen by config.json.  `spec_hook`, when given,
    takes the architecture's ModelSpec and returns the one to build (a run-time option that changes a part's
    parameters, such as a sliding window for every attention layer)."""
    arch, cfg = load_config(folder)
    spec = arch.build_spec(cfg)
    if spec_hook is not None:
        spec = spec_hook(spec)
    probe = DecoderModel(spec)                       # host-only: lists the tensors the model reads
    t0 = time.time()
    tensors = load_tensors(folder, probe.tensor_specs())
    model = build_model(spec, tensors, dtype, device, verbose)
    if verbose:
        print(f"[tnx-b200] {arch.name} loaded from {folder} as {canonical_dtype(dtype)} in "
              f"{time.time() - t0:.1f} s ({model.parameter_bytes() / 1e9:.2f} GB of weights)",
              file=sys.stderr, flush=True)
    return model, cfg
