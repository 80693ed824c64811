"""Reading a model folder's config.json as a plain dictionary.

Nothing here knows an architecture: the dictionary goes to the registry, which picks the
architecture by ``architectures[0]`` and hands it the same dictionary to parse.  The reference
goes through ``AutoConfig`` with a raw-JSON shim for unknown model types
(python/freetoken/utils/hf.py:132-204); this engine reads the file itself.
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict

from ..errors import ConfigError


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: config.json must hold a JSON object")
    return raw
