"""Every name listed in docs/API_MAP.md is importable from the module its section names."""
import importlib
import re
from pathlib import Path


def test_api_map_names_exist():
    text = (Path(__file__).resolve().parents[1] / "docs" / "API_MAP.md").read_text()
    sections = re.split(r"^## ", text, flags=re.M)[1:]
    assert len(sections) >= 40
    total = 0
    for sec in sections:
        head, _, body = sec.partition("\n")
        mod = re.search(r"`([\w.:]+)`", head).group(1)
        m = importlib.import_module(mod.split(":")[0])
        if ":" in mod:
            m = getattr(m, mod.split(":")[1])
        names = re.findall(r"`(\w+)`", body.split("\n\n", 2)[1] if "\n\n" in body else body)
        assert names, head
        for n in names:
            assert hasattr(m, n), f"{mod}.{n}"
        total += len(names)
    assert total > 1650
