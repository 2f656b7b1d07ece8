"""Every bounded-wait site code of the CUDA sources has a description on the host side."""
import re
from pathlib import Path

from causal_trainer_dev_b200.ops import lib


def test_every_site_code_is_described():
    csrc = Path(lib.__file__).resolve().parent / "csrc"
    codes = {}
    for path in sorted(csrc.iterdir()):
        if path.suffix in (".cu", ".cuh", ".h"):
            for name, value in re.findall(r"\b(SITE_[A-Z0-9_]+)\s*=\s*(0x[0-9a-fA-F]+)", path.read_text()):
                where = f"{path.name}:{name}"
                assert int(value, 16) not in codes, f"{where} reuses the code of {codes[int(value, 16)]}"
                codes[int(value, 16)] = where
    assert codes, "no site codes found"
    missing = {hex(c): where for c, where in codes.items() if c not in lib._SITES}
    assert not missing, missing
