"""The operator module can be imported the way the reference's hosts import it:
as a top-level `deploy_step` found through operator_dir()."""
import subprocess
import sys


def test_deploy_step_imports_as_a_top_level_module():
    code = ("import sys, token2tile_b200; sys.path.insert(0, token2tile_b200.operator_dir()); "
            "import deploy_step; assert hasattr(deploy_step, 'MaskedStepDeploy') and hasattr(deploy_step, 'online_u'); "
            "print('ok')")
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr
