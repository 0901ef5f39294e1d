import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); deselect with -m 'not gpu'")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Random-weight model folders of the tiny configurations, made once per run in a
    temporary folder."""
    import helpers
    made = {}

    def get(name: str) -> str:
        if name not in made:
            made[name] = helpers.make_model_dir(str(tmp_path_factory.mktemp(f"model_{name}")), name)
        return made[name]
    return get


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    from plain.hunyuan_plain import PlainModel
    made = {}

    def get(name: str):
        if name not in made:
            made[name] = PlainModel(model_dirs(name))
        return made[name]
    return get
