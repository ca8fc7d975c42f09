"""Import helper for the golden-vector generator: makes the upstream P2 package importable
in a container that lacks hydra/omegaconf, without writing any file next to it.

Only `make_golden.py` uses this module, and only on a machine where the upstream checkout
is mounted (path taken from the P2_REFERENCE_SRC environment variable).  Nothing in the
product, the oracle or the tests imports it at run time.
"""
from __future__ import annotations

import os
import sys
import types


def install(reference_src: str | None = None) -> None:
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    src = reference_src or os.environ.get("P2_REFERENCE_SRC")
    if not src or not os.path.isdir(src):
        raise SystemExit("set P2_REFERENCE_SRC to the `src` directory of the upstream checkout")
    if src not in sys.path:
        sys.path.insert(0, src)
    if "hydra" not in sys.modules:
        hydra = types.ModuleType("hydra")
        hydra.main = lambda *a, **k: (lambda f: f)
        core = types.ModuleType("hydra.core")
        store = types.ModuleType("hydra.core.config_store")

        class ConfigStore:
            _inst = None

            @classmethod
            def instance(cls):
                if cls._inst is None:
                    cls._inst = cls()
                return cls._inst

            def store(self, *a, **k):
                return None

        store.ConfigStore = ConfigStore
        hydra.core = core
        core.config_store = store
        sys.modules["hydra"] = hydra
        sys.modules["hydra.core"] = core
        sys.modules["hydra.core.config_store"] = store
    if "omegaconf" not in sys.modules:
        oc = types.ModuleType("omegaconf")

        class DictConfig(dict):
            pass

        class OmegaConf:
            @staticmethod
            def to_container(c, resolve=True):
                return dict(c)

        oc.DictConfig = DictConfig
        oc.OmegaConf = OmegaConf
        sys.modules["omegaconf"] = oc
