"""Makes the golden logits under tests/golden/ from the reference's own Python model
(AustinJiangg/nanoinfer, nanoinfer/model.py) on the CPU.

    PYTHONPATH=<reference checkout>:<this repo> python tests/golden/make_golden.py

For each tiny configuration it writes a random model folder with this engine's random-weights
mode (seed below) into a temporary folder, loads those tensors into the reference's ``Model``
(names = checkpoint names minus ``model.``, nanoinfer/weights.py:92-97; a tied head is assigned the
embedding as nanoinfer/weights.py:167-169 does), runs whole sequences without a cache, and stores
ids and float32 logits in ``<name>.npz``. The tests rebuild the same model folder from the seed
and compare the plain implementation (tests/plain_qwen2.py) with these logits.
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tiny_configs import TINY_A, TINY_B  # noqa: E402
from plain_qwen2 import read_weights  # noqa: E402
from nanoinfer_b200.registry import config_from_json_dict  # noqa: E402
from nanoinfer_b200.weights import write_random_model  # noqa: E402

from nanoinfer.config import ModelConfig  # noqa: E402  (the reference)
from nanoinfer.model import Model  # noqa: E402

SEED = 1234
LENGTHS = {"A": [1, 7, 33], "B": [2, 9, 40]}


def main():
    for name, cfg_json in (("A", TINY_A), ("B", TINY_B)):
        cfg = config_from_json_dict(cfg_json)
        with tempfile.TemporaryDirectory() as d:
            write_random_model(cfg, d, seed=SEED, dtype="float32")
            w = read_weights(d, torch.float32)
        rcfg = ModelConfig(
            vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
            num_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, rms_norm_eps=cfg.rms_norm_eps,
            rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
            tie_word_embeddings=cfg.tie_word_embeddings)
        model = Model(rcfg).eval()
        sd = {k[len("model."):] if k.startswith("model.") else k: v for k, v in w.items()}
        if cfg.tie_word_embeddings and "lm_head.weight" not in sd:
            sd["lm_head.weight"] = sd["embed_tokens.weight"]
        missing, unexpected = model.load_state_dict(sd, strict=False)
        assert not [m for m in missing if not m.startswith("rope_")] and not unexpected, (missing, unexpected)
        g = torch.Generator().manual_seed(99)
        out = {}
        for i, n in enumerate(LENGTHS[name]):
            ids = torch.randint(0, cfg.vocab_size, (n,), generator=g)
            with torch.no_grad():
                logits = model(ids[None])[0]
            out[f"ids{i}"] = ids.numpy().astype(np.int32)
            out[f"logits{i}"] = logits.numpy().astype(np.float32)
        np.savez_compressed(os.path.join(HERE, f"qwen2_tiny_{name}.npz"), seed=SEED, **out)
        print(name, "ok", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
