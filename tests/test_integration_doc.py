"""The integration guide shows the reference-side binding; the text it shows is the text of the file the GPU test
executes (spio_b200/examples/reference_binding.py), line for line."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_binding_shown_in_the_document_is_the_executed_file():
    doc = (ROOT / "INTEGRATION.md").read_text()
    block = re.search(r"```python\n(_lib = ctypes.*?)```", doc, re.S).group(1)
    source = {line.strip() for line in (ROOT / "spio_b200" / "examples" / "reference_binding.py").read_text().splitlines()}
    shown = [line.strip() for line in block.splitlines() if line.strip()]
    assert len(shown) > 25
    missing = [line for line in shown if line not in source]
    assert not missing, missing
