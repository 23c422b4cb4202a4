#!/usr/bin/env python
"""Copy the first N training shards (and the whole validation split) of a prepared dataset into a smaller
dataset folder with a matching manifest — for quick runs and uploads.

    python scripts/make_data_subset.py --src data/nemotron_cc --dst data/nemotron_cc_1shard --shards 1
"""

import argparse
import json
import shutil
from pathlib import Path


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--src", type=Path, required=True)
    ap.add_argument("--dst", type=Path, required=True)
    ap.add_argument("--shards", type=int, default=1)
    a = ap.parse_args(argv)
    manifest = json.loads((a.src / "manifest.json").read_text())
    a.dst.mkdir(parents=True, exist_ok=True)
    train = manifest["splits"]["train"]["shards"][: a.shards]
    manifest["splits"]["train"] = {"n_tokens": sum(s["n_tokens"] for s in train), "shards": train}
    for split in manifest["splits"].values():
        for s in split["shards"]:
            shutil.copy2(a.src / s["path"], a.dst / s["path"])
    manifest["subset_of"] = str(a.src)
    (a.dst / "manifest.json").write_text(json.dumps(manifest, indent=2))
    print({k: v["n_tokens"] for k, v in manifest["splits"].items()})


if __name__ == "__main__":
    main()
