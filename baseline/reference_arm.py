"""Reference arm of the headline benchmark.

The reference (KellyKinyama/dart-pytorch) is a Dart package: it has no ``setup.py`` / ``pyproject.toml``, so
``pip install --target baseline/_ref`` of its tree fails ("Neither 'setup.py' nor 'pyproject.toml' found"), and no Dart SDK
exists on the build or GPU machines, so its public API (Dart classes over ``dart:ffi``) cannot be executed.  The arm
therefore reports itself unavailable."""
from __future__ import annotations

import json


def run(args, metric, model_cfg, seq):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Dart package (no setup.py/pyproject.toml: pip install fails) and no Dart SDK "
                       "is present, so its public API cannot run GPT-2 124M training here",
        "metric": metric, "n_gpus": args.gpus}))
