"""Alias of ``picotron_b200.parallel.deepep_backend`` under the reference's import path."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("picotron_b200.parallel.deepep_backend")
