#!/usr/bin/env python3
"""Collects the reference's golden vectors for the optimizer-step path.

Reads the PyTorch-generated fixtures the reference keeps for its own tests
(testdata/sgd.json, testdata/param_groups.json, testdata/nn_conv_step.json) and
writes the subset that pins this path into ``tests/golden/optimizer_vectors.json``.
The reference checkout is only needed to run this script; the tests read the
committed output.

    python tests/golden/make_golden.py --reference /path/to/gograd
"""
import argparse
import json
from pathlib import Path


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", type=Path, required=True, help="path of a gograd checkout")
    ap.add_argument("--output", type=Path, default=Path(__file__).resolve().parent / "optimizer_vectors.json")
    args = ap.parse_args()
    td = args.reference / "testdata"
    sgd = json.loads((td / "sgd.json").read_text())
    groups = json.loads((td / "param_groups.json").read_text())
    conv = json.loads((td / "nn_conv_step.json").read_text())
    out = {
        "provenance": {
            "sgd": "testdata/sgd.json (tools/gen_sgd_fixture.py; read by autograd/sgd_test.go:53-125)",
            "param_groups": "testdata/param_groups.json (tools/gen_param_groups_fixture.py; read by "
                            "autograd/param_groups_test.go:86-198)",
            "clip_adamw_step": "testdata/nn_conv_step.json (tools/gen_nn_fixture.py:33-36: clip_grad_norm_(0.8) "
                               "then one AdamW(lr=.003, weight_decay=.01) step); fields parameters/gradients/updated",
            "torch_version": {"sgd": sgd["torch_version"], "param_groups": groups["torch_version"]},
        },
        "tolerances": {
            "values": {"atol": 5e-7, "rtol": 3e-6, "source": "autograd/sgd_test.go:89-93"},
            "adamw_v": {"atol": 5e-8, "rtol": 3e-7, "source": "autograd/param_groups_test.go:185-186"},
        },
        "sgd": [
            {"name": c["name"], "options": c["options"], "initial": c["initial"],
             "steps": [{"lr": s["lr"], "gradients": s["gradients"], "values": s["values"], "buffers": s["buffers"]}
                       for s in c["steps"]]}
            for c in sgd["cases"]
        ],
        "param_groups": [
            {"name": c["name"], "kind": c["kind"], "params": c["params"], "groups": c["groups"],
             "steps": [{k: s[k] for k in ("gradients", "values", "buffers", "moments") if k in s}
                       for s in c["steps"]]}
            for c in groups["cases"]
        ],
        "clip_adamw_step": {
            "max_norm": 0.8, "lr": 0.003, "weight_decay": 0.01,
            "names": list(conv["parameters"].keys()),
            "parameters": conv["parameters"], "gradients": conv["gradients"], "updated": conv["updated"],
        },
    }
    args.output.write_text(json.dumps(out, separators=(",", ":")) + "\n", encoding="utf-8")
    print(f"{args.output}: {len(out['sgd'])} sgd cases, {len(out['param_groups'])} group cases, "
          f"{sum(len(v) for v in conv['parameters'].values())} clip+adamw parameters")


if __name__ == "__main__":
    main()
