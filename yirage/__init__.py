"""`import yirage` resolves to the B200-native package, so scripts written against the
reference (demo/llama3/demo.py, benchmark/rmsnorm.py) run unchanged."""
import sys

import yirage_b200 as _impl
from yirage_b200 import *  # noqa: F401,F403
from yirage_b200 import __version__  # noqa: F401

for _name in ("core", "kernel", "lowering", "persistent_kernel", "speculative", "threadblock",
              "utils", "global_config", "version", "profiler_persistent"):
    try:
        _mod = __import__(f"yirage_b200.{_name}", fromlist=[_name])
    except ImportError:
        continue
    sys.modules[f"yirage.{_name}"] = _mod
    globals()[_name] = _mod
