"""pytest configuration: registers the `gpu` marker and puts the repository root first on sys.path,
ahead of any unrelated `flash_attn_2_cuda` that may be installed in site-packages."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT in sys.path:
    sys.path.remove(ROOT)
sys.path.insert(0, ROOT)
sys.path.insert(1, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
