"""config.json files of the family's published sizes (the layer sizes of Llama 3.2 1B, 3.2 3B and
3.1 8B), for random-weight models and measurements.  They are data, read like any other
config.json; nothing in the package depends on them.

The reference fixes such numbers in code instead: rope theta 500000 and the llama3 scaling
(32, 1, 4, 8192), eps 1e-5, bos 128000 and eos 128001 in src/model/model.cpp:150-162, the sizes in
the header of its own weight file (include/nanoinfer/model/config.h:13-21).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))


def preset_names() -> List[str]:
    return sorted(f[:-5] for f in os.listdir(_HERE) if f.endswith(".json"))


def preset(name: str) -> Dict:
    """The config.json dictionary of a named size; raises KeyError listing the names there are."""
    path = os.path.join(_HERE, name + ".json")
    if not os.path.isfile(path):
        raise KeyError(f"no preset {name!r}; there are: {', '.join(preset_names())}")
    with open(path) as f:
        return json.load(f)
