"""Writes the two small weight directories under ``tests/golden/bank_files/`` with the REFERENCE's own writer
(``freetoken.checkpoint.ftw.FTWWriter``), so that the reader of this package is tested against bytes it did not
produce.  Run once in a container that has the reference checkout:

    python tests/golden/make_bank_files.py /path/to/reference/freetoken/python

The tensors are seeded (``bank_layers`` below is imported by the tests to regenerate them)."""
import pathlib
import shutil
import sys

import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

LAYERS, EXPERTS, HIDDEN, INTER = 3, 4, 64, 32
SHARD_LIMIT = 16384
STORED = ("gate_up_packed", "gate_up_scale", "gate_up_global", "down_packed", "down_scale", "down_global")
ROLES = ("gate_up", "gate_up_scale", "gate_up_global", "down", "down_scale", "down_global")


def bank_layers():
    from qwen36_moe_16gb_b200 import synth

    shape = synth.Shape(hidden=HIDDEN, intermediate=INTER, num_experts=EXPERTS, top_k=2, shared_intermediate=64)
    g = torch.Generator().manual_seed(2024)
    layers = []
    for l in range(LAYERS):
        b = synth.make_banks(g, shape)
        b["gate_up_global"] = b["gate_up_global"] * (1 + l) + torch.arange(2 * INTER) * 1e-4
        b["down_global"] = b["down_global"] * (2 + l) + torch.arange(HIDDEN) * 1e-4
        layers.append(b)
    return layers


def dense_extras():
    g = torch.Generator().manual_seed(7)
    return {"model.norm.weight": torch.randn(HIDDEN, generator=g).bfloat16(), "model.scalar": torch.tensor(0.5)}


def main(ref_python: str) -> None:
    sys.path.insert(0, ref_python)
    from freetoken.checkpoint.ftw import FTWWriter, layer_bank_entry_name

    layers = bank_layers()
    for form in ("per_layer", "flat"):
        out = HERE / "bank_files" / form
        if out.exists():
            shutil.rmtree(out)
        w = FTWWriter(str(out), shard_limit=SHARD_LIMIT)
        for name, t in dense_extras().items():
            w.add_tensor(name, t, "weight")
        for role, stored in zip(ROLES, STORED):
            if form == "per_layer":
                for l in range(LAYERS):
                    w.add_tensor(layer_bank_entry_name(stored, l), layers[l][role], "experts_bank")
            else:
                w.add_tensor(stored, torch.cat([b[role] for b in layers]), "experts_bank")
        w.finalize({"quant_format": "nvfp4", "expert_bank_num_layers": LAYERS})
        print(form, sum(f.stat().st_size for f in out.iterdir()), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
