"""``stitch-mtp``: put a trained native MTP draft back into a Target checkpoint directory - the draft's tensors are
written under the Target's own ``mtp.*`` keys into one new safetensors shard and the weight index is updated, so a
serving engine that reads native MTP heads picks the trained one up (reference: aspec/commands/stitch_native_mtp.py)."""
from __future__ import annotations

import argparse
import json
import os
import sys


def stitch(asset_dir: str, target_dir: str, output_dir: str, shard_name: str = "model-mtp-trained.safetensors") -> dict:
    from safetensors.torch import load_file, save_file
    manifest = json.load(open(os.path.join(asset_dir, "export_manifest.json")))
    if manifest.get("algorithm") != "mtp":
        raise ValueError("stitch-mtp needs an exported native MTP draft")
    tensors = load_file(os.path.join(asset_dir, "model.safetensors"))
    native = {k: v for k, v in tensors.items() if k.startswith("mtp.")}
    if not native:
        raise ValueError("the asset holds no mtp.* tensors")
    if os.path.abspath(output_dir) == os.path.abspath(target_dir):
        raise ValueError("refusing to modify the Target checkpoint in place; choose another output directory")
    os.makedirs(output_dir, exist_ok=False)
    index_path = os.path.join(target_dir, "model.safetensors.index.json")
    index = json.load(open(index_path)) if os.path.isfile(index_path) else {"metadata": {}, "weight_map": {}}
    replaced = sorted(k for k in native if k in index["weight_map"])
    for name in os.listdir(target_dir):
        src = os.path.join(target_dir, name)
        if os.path.isfile(src) and name != "model.safetensors.index.json":
            os.symlink(os.path.abspath(src), os.path.join(output_dir, name))
    save_file({k: v.contiguous() for k, v in native.items()}, os.path.join(output_dir, shard_name))
    for k in native:
        index["weight_map"][k] = shard_name
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2, sort_keys=True)
    report = {"output_dir": output_dir, "tensors": len(native), "replaced_existing": len(replaced), "shard": shard_name}
    with open(os.path.join(output_dir, "stitch_manifest.json"), "w") as f:
        json.dump({**report, "asset": os.path.abspath(asset_dir), "target": os.path.abspath(target_dir)}, f, indent=2)
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 stitch-mtp", description=__doc__)
    ap.add_argument("--asset-dir", required=True, help="directory written by `aspec-b200 export`")
    ap.add_argument("--target-dir", required=True)
    ap.add_argument("--output-dir", required=True)
    a = ap.parse_args(argv)
    print(json.dumps(stitch(a.asset_dir, a.target_dir, a.output_dir), indent=2))
    return 0


if __name__ == "__main__":
    sys.exit(main())
