import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_assets(tmp_path_factory):
    """Tiny dense GQA checkpoint (fp32, seed 0) compiled for the CPU backend."""
    from plow_b200 import plowc
    from plow_b200.models import config, reference
    d = tmp_path_factory.mktemp("tiny")
    cfg = config.tiny_dense_config()
    reference.write_checkpoint(cfg, d / "ckpt", seed=0)
    plowc.compile_dir(d / "ckpt", d / "assets", arch="cpu", n_cu=8, max_rows=256, decode_rungs=[1, 2, 4, 8], max_seqs=8)
    return d


@pytest.fixture(scope="session")
def tiny_reference(tiny_assets):
    import glob
    from safetensors.torch import load_file
    from plow_b200.models import config, reference
    state = {}
    for f in glob.glob(str(tiny_assets / "ckpt" / "*.safetensors")):
        state.update(load_file(f))
    return reference.ReferenceModel(config.spec_from_config(config.tiny_dense_config()), state)
