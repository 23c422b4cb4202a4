#!/usr/bin/env bash
# Publish a prepared token dataset (the *.bin shards and manifest.json that `python -m nanonemo_b200.data.prepare` wrote) as a
# PRIVATE Kaggle dataset, so that a notebook session can mount it instead of downloading and tokenising again.
#
#   scripts/publish_dataset.sh data/nemotron_cc my-token-shards
#
# Before anything is uploaded every shard is checked against the sha256 recorded in the manifest (a truncated or stale shard
# must not become the published copy). Only shards and the manifest are staged, through hard links, never raw downloads.
# Credentials: KAGGLE_API_TOKEN, or ~/.kaggle/access_token, or the legacy ~/.kaggle/kaggle.json. Needs the `kaggle` CLI and
# network access, neither of which exists on the build machines of this repository: there the script stops at the first check.
set -euo pipefail

data_dir=${1:?usage: scripts/publish_dataset.sh <data_dir> <dataset-slug>}
slug=${2:?usage: scripts/publish_dataset.sh <data_dir> <dataset-slug>}
command -v kaggle >/dev/null 2>&1 || { echo "the kaggle CLI is not installed" >&2; exit 3; }
[ -f "$data_dir/manifest.json" ] || { echo "$data_dir/manifest.json not found: run the prepare step first" >&2; exit 2; }

python - "$data_dir" <<'PY'
import json, sys
from pathlib import Path
sys.path.insert(0, str(Path(__file__).resolve().parent if "__file__" in globals() else Path.cwd()))
sys.path.insert(0, str(Path.cwd()))
from nanonemo_b200.data.shard import file_sha256, read_header
root = Path(sys.argv[1])
manifest = json.loads((root / "manifest.json").read_text())
bad = 0
for split, info in manifest["splits"].items():
    for shard in info["shards"]:
        path = root / shard["path"]
        read_header(path)  # magic, version, exact size
        if "sha256" in shard and file_sha256(path) != shard["sha256"]:
            print(f"checksum mismatch: {path}", file=sys.stderr)
            bad += 1
print(f"verified {sum(len(i['shards']) for i in manifest['splits'].values())} shards, {bad} bad")
sys.exit(1 if bad else 0)
PY

owner=$(python -c "
from kaggle.api.kaggle_api_extended import KaggleApi
api = KaggleApi(); api.authenticate(); print(api.config_values['username'])")
stage="$data_dir/.publish_stage"
rm -rf "$stage"
mkdir -p "$stage"
ln "$data_dir"/*.bin "$data_dir"/manifest.json "$stage"/
printf '{\n  "title": "%s",\n  "id": "%s/%s",\n  "licenses": [{"name": "other"}]\n}\n' "$slug" "$owner" "$slug" > "$stage/dataset-metadata.json"
if kaggle datasets status "$owner/$slug" >/dev/null 2>&1; then
    kaggle datasets version --path "$stage" --message "refresh shards"
else
    kaggle datasets create --path "$stage"
fi
rm -rf "$stage"
