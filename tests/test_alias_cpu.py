"""The ``rwkvtune`` import alias: unmodified reference-style imports resolve to this package."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code: str, *args):
    env = dict(os.environ, PYTHONPATH=ROOT)
    return subprocess.run([sys.executable, *args], input=code, capture_output=True, text=True, env=env, cwd=ROOT,
                          timeout=300)


def test_script_with_reference_imports_runs_through_the_alias(tmp_path):
    script = tmp_path / "user_script.py"
    script.write_text(textwrap.dedent("""
        import sys
        from rwkvtune import AutoModel, AutoTokenizer, SFTConfig, SFTTrainer, GRPOConfig, GRPOTrainer, LoraConfig
        from rwkvtune.peft import get_peft_model
        from rwkvtune.models.rwkv7 import RWKV7Model
        from rwkvtune.inference import GRPOBatchGenerator, TokenSampler
        from rwkvtune.training.grpo.loss import DAPOLoss
        import rwkvtune, rwkvtune_b200
        assert rwkvtune.AutoModel is rwkvtune_b200.AutoModel
        assert sys.modules["rwkvtune.peft"] is sys.modules["rwkvtune_b200.peft"]
        print("alias ok", sys.argv[1])
    """))
    res = subprocess.run([sys.executable, "-m", "rwkvtune_b200.alias", str(script), "arg1"], capture_output=True,
                         text=True, env=dict(os.environ, PYTHONPATH=ROOT), cwd=str(tmp_path), timeout=300)
    assert res.returncode == 0, res.stderr
    assert "alias ok arg1" in res.stdout


def test_alias_refuses_to_shadow_a_real_rwkvtune(tmp_path):
    fake = tmp_path / "site" / "rwkvtune"
    fake.mkdir(parents=True)
    (fake / "__init__.py").write_text("REAL = True\n")
    code = textwrap.dedent(f"""
        import sys
        sys.path.insert(0, {str(tmp_path / 'site')!r})
        import rwkvtune_b200.alias as alias
        try:
            alias.install()
        except alias.AliasConflict as exc:
            print("refused")
        import rwkvtune
        assert rwkvtune.REAL
    """)
    res = _run(code, "-")
    assert res.returncode == 0, res.stderr
    assert "refused" in res.stdout


def test_install_is_idempotent_and_reversible():
    code = textwrap.dedent("""
        import sys
        import rwkvtune_b200.alias as alias
        alias.install(); alias.install()
        import rwkvtune.sampling_params as sp
        assert sp.SamplingParams is __import__("rwkvtune_b200.sampling_params", fromlist=["x"]).SamplingParams
        alias.uninstall()
        assert not alias.installed() and "rwkvtune" not in sys.modules
        print("ok")
    """)
    res = _run(code, "-")
    assert res.returncode == 0, res.stderr
