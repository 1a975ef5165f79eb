"""Model-folder reader and family registry, as far as they go without a GPU."""
import json
import os

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md


def make(tmp_path, cfg, tensors=None):
    return md.write_model_dir(str(tmp_path / "m"), cfg, tensors if tensors is not None else {"embed": np.zeros((4, 8), np.float32)})


def test_unknown_architecture_is_named(tmp_path):
    p = make(tmp_path, {"architecture": "Nonesuch"})
    with pytest.raises(E.NB200Error, match="unknown architecture \"Nonesuch\""):
        E.Engine(p, 16)


def test_broken_folders_are_reported(tmp_path):
    with pytest.raises(E.NB200Error, match="cannot read"):
        E.Engine(str(tmp_path), 16)
    p = make(tmp_path, {"architecture": "Famudra"})
    open(os.path.join(p, "config.json"), "w").write('{"architecture": ')
    with pytest.raises(E.NB200Error, match="config.json"):
        E.Engine(p, 16)
    open(os.path.join(p, "config.json"), "w").write(json.dumps({"architecture": "Famudra"}))
    with open(os.path.join(p, "model.safetensors"), "r+b") as f:
        f.write((1 << 40).to_bytes(8, "little"))
    with pytest.raises(E.NB200Error, match="header length"):
        E.Engine(p, 16)


@pytest.mark.skipif(E.device_count() > 0, reason="box has a GPU")
def test_no_cpu_fallback_for_model_folders(tmp_path):
    cfg = md.famudra_config(16, 8, [("rglru", {"width": 8, "blocks": 1, "conv": 2}, None)])
    p = md.write_model_dir(str(tmp_path / "f"), cfg, md.famudra_random(cfg))
    with pytest.raises(E.NB200Error, match="no CUDA device"):
        E.Engine(p, 16)


def test_bf16_writer_rounds_to_nearest_even():
    a = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 0.0], np.float32)     # 1 + 2^-8 is a tie: even mantissa wins
    r = md.bf16_round(a)
    assert r[0] == 1.0 and r[1] == 1.0 and r[2] == np.float32(1.015625) and abs(r[3] + 3.140625) < 1e-6
