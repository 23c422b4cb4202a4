"""The node notebook only launches files of the repository: every script, config and module it names must exist."""

import json
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def test_notebook_cells_reference_existing_files():
    nb = json.loads((ROOT / "notebooks" / "b200_node.ipynb").read_text())
    assert nb["nbformat"] == 4
    text = "\n".join("".join(c["source"]) if isinstance(c["source"], list) else c["source"] for c in nb["cells"] if c["cell_type"] == "code")
    named = set(re.findall(r"(?:scripts|configs|tests)/[\w/.$-]+\.(?:py|sh|yaml)", text)) | {"bench.py", "__graft_entry__.py"}
    assert len(named) >= 10
    for rel in named:
        if "$" in rel:  # a shell loop variable: check every expansion the loop lists
            stem, var = rel.split("$", 1)
            loop = re.search(r"for \w+ in ([^;]+); do[^\n]*\n?[^\n]*" + re.escape(stem), text)
            assert loop, rel
            for value in loop.group(1).split():
                assert (ROOT / (stem + value + rel[rel.index("$") + 1 + len(re.match(r"\w+", var).group()):])).exists(), (rel, value)
        else:
            assert (ROOT / rel).exists(), rel
