"""Every example launch script must only use configuration keys that exist."""
import glob
import os
import re

from skyrl_b200.config.config import SkyRLTrainConfig
from skyrl_b200.config.sft_config import SFTConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _overrides(path):
    out = []
    for line in open(path):
        line = line.strip().rstrip("\\").strip()
        if re.match(r"^[a-z_][a-z0-9_.]*=", line):
            line = re.sub(r"\$\{[A-Z_]+:-([^}]*)\}", r"\1", line)
            line = line.replace("$MODEL", "tiny-llama").replace("$DATA", "/tmp/d").replace("$HOME", "/tmp").replace("$NGPU", "1")
            out.append(line)
    return out


def test_example_scripts_parse():
    scripts = sorted(glob.glob(os.path.join(ROOT, "examples", "**", "*.sh"), recursive=True))
    assert len(scripts) >= 25
    for s in scripts:
        ov = _overrides(s)
        assert ov, s
        text = open(s).read()
        if "entrypoints.main_sft" in text:
            SFTConfig.from_cli_overrides(ov)
        else:
            SkyRLTrainConfig.from_cli_overrides(ov)


def test_custom_registrations_import():
    import importlib

    from skyrl_b200.algorithms import rl

    importlib.import_module("examples.algorithms.custom_advantage_estimator")
    importlib.import_module("examples.algorithms.custom_policy_loss")
    assert rl.AdvantageEstimatorRegistry.get("centered_reward") is not None
    assert rl.PolicyLossRegistry.get("capped_reinforce") is not None
