"""The `oops` import path: with compat/ on PYTHONPATH the reference's names resolve to this library."""

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_import_oops_resolves_to_this_library():
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(ROOT / "compat"), str(ROOT)]))
    code = ("import oops, oops_b200; assert oops.triangle_attention is oops_b200.triangle_attention; "
            "assert oops.OOpsUnsupportedError is oops_b200.OOpsUnsupportedError; "
            "assert not hasattr(oops, 'token_mask_from_msa_mask'); print('ok')")
    done = subprocess.run([sys.executable, "-c", code], env=env, cwd="/", capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and done.stdout.strip() == "ok", done.stderr
