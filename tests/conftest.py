import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{name: folder} of the tiny random models, written once per session in a temporary folder."""
    from configs import CONFIGS
    from iitj_llm_coopt_b200.weights import write_model_dir
    out = {}
    for name, (cfg, seed, _page) in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_model_dir(cfg, str(d), seed)
        out[name] = str(d)
    return out


@pytest.fixture(params=["tma", "cp_async"])
def decode_loads(request):
    """Both decode attention kernels: keys and values fetched by TMA (pages of 8 to 64 tokens), or copied by the
    threads themselves (any page size)."""
    from iitj_llm_coopt_b200 import kernels
    K = kernels.load()
    before = K.decode_tma
    K.decode_tma = request.param == "tma"
    yield request.param
    K.decode_tma = before
