"""Layer-shape helpers with the names quant.py imports from src.model_utils
(src/model_utils.py:8-29)."""
from __future__ import annotations

import math
import re
from typing import Dict, Sequence, Union

import torch.nn as nn

LINEAR_LAYERS = (nn.Linear,)


def get_number_of_rows_and_cols(layer: nn.Module):
    """(out_features, product of the remaining weight dims): src/model_utils.py:11-12."""
    shape = layer.weight.shape
    return int(shape[0]), int(math.prod(shape[1:]))


def select_layers(model: nn.Module, layer_prefix: str = "", layer_regex: str = ".*",
                  layer_classes: Union[type, Sequence[type]] = nn.Module) -> Dict[str, nn.Module]:
    """Named sub-modules of the given classes whose name starts with the prefix and
    matches the regex (src/model_utils.py:15-29)."""
    classes = tuple(layer_classes) if isinstance(layer_classes, (list, tuple)) else layer_classes
    pattern = re.compile(layer_regex)
    return {
        name: module
        for name, module in model.named_modules()
        if isinstance(module, classes) and name.startswith(layer_prefix or "") and pattern.search(name)
    }
