#!/usr/bin/env python3
"""Golden vectors for exact key-bias removal, made by the reference's own ``rotated_bias``.

    python tests/golden/make_bias_golden.py /path/to/PITCH

Imports ``reference/mechanism_eval.py`` unchanged and calls its ``rotated_bias(module, key)``
(lines 82-91) and ``rope_parts`` (lines 74-79).  The reference applies them inside a loaded
language model; here the model is a stand-in that carries exactly what those two functions touch:
a key-projection bias, the head dimension, the rotary embedding of the ``transformers`` Qwen2
implementation (random-initialised, no checkpoint: it has no weights, only the frequency table)
and that implementation's ``rotate_half``.  Written to ``tests/golden/rotated_bias.npz``:
per case the bias ``[heads, dim]``, the model's cos / sin tables ``[T, dim]`` and the reference's
``R_t b`` ``[heads, T, dim]``, all float32.
"""
import json
import sys
import types
from pathlib import Path

import numpy as np

sys.dont_write_bytecode = True
HERE = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    sys.path.insert(0, str(Path(ref_root) / "reference"))
    import torch
    import mechanism_eval as M                      # the reference module, unchanged
    from transformers import Qwen2Config
    from transformers.models.qwen2 import modeling_qwen2 as Q

    arrays, cases = {}, []
    gen = torch.Generator().manual_seed(20241)
    for name, heads, dim, T, theta in (("qwen64", 2, 64, 300, 1000000.0), ("llama128", 8, 128, 96, 500000.0),
                                       ("small8", 1, 8, 40, 10000.0)):
        cfg = Qwen2Config(hidden_size=heads * dim, num_attention_heads=heads, num_key_value_heads=heads, head_dim=dim,
                          rope_theta=theta, max_position_embeddings=4096)
        rotary = Q.Qwen2RotaryEmbedding(cfg)

        class Stub:                                  # what rotated_bias / rope_parts read from an attention module
            pass
        Stub.__module__ = Q.__name__                 # rope_parts looks rotate_half up in the module's own file
        module = Stub()
        module.head_dim = dim
        module.k_proj = types.SimpleNamespace(bias=torch.randn(heads * dim, generator=gen) * 3.0)
        M.MODEL["m"] = types.SimpleNamespace(model=types.SimpleNamespace(rotary_emb=rotary))
        key = torch.zeros(1, heads, T, dim, dtype=torch.float32)
        rb = M.rotated_bias(module, key)             # (1, heads, T, dim)
        cos, sin, _ = M.rope_parts(module, T, torch.float32, "cpu")    # (1, 1, T, dim)
        arrays[f"{name}/bias"] = module.k_proj.bias.view(heads, dim).numpy().astype(np.float32)
        arrays[f"{name}/cos"] = cos[0, 0].numpy().astype(np.float32)
        arrays[f"{name}/sin"] = sin[0, 0].numpy().astype(np.float32)
        arrays[f"{name}/rotated_bias"] = rb[0].numpy().astype(np.float32)
        cases.append(dict(key=name, heads=heads, dim=dim, positions=T, rope_theta=theta))
    arrays["__cases__"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "rotated_bias.npz", **arrays)
    print(f"wrote {HERE / 'rotated_bias.npz'}: {len(cases)} cases")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_bias_golden.py <path to the reference checkout>")
    main(sys.argv[1])
