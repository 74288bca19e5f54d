"""Place the reference's own Python layer beside the oracle, for the drop-in test.

    python oracle/fetch_ref_interface.py <path to the reference checkout>

Copies ``flex_block_attn/flex_block_attn_interface.py`` (the reference's autograd Function and
``flex_block_attn_func``, which import ``attn_forward`` / ``attn_backward`` from the compiled module
``flex_block_attn_cuda``) byte for byte into ``oracle/_ref/``.  That directory is not part of the
repository's history: the file is the reference's source, used only by tests/test_dropin_gpu.py to
show that the reference's unmodified Python layer runs on top of this library when
``flex_block_attn_cuda`` is replaced by ``flex_block_attn_b200.compat``.  TEST INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref" / "flex_block_attn_interface.py"


def fetch(reference_root: Path) -> Path:
    src = Path(reference_root) / "flex_block_attn" / "flex_block_attn_interface.py"
    if not src.exists():
        raise FileNotFoundError(src)
    DEST.parent.mkdir(parents=True, exist_ok=True)
    shutil.copyfile(src, DEST)
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(fetch(Path(sys.argv[1])))
