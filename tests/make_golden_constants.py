"""Constants of tests/golden/make_golden.py, importable without triggering its reference imports."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden'))
from make_golden import INF_STEP, OPTIM_CFG, OPTIM_CHUNK, OPTIM_HYPER, OPTIM_STEPS    # noqa: E402,F401
