#!/usr/bin/env python
"""Train a speculative-decoding draft model.

    python scripts/train.py --verifier-name-or-path <dir> --data-path <dir> [flags]
    torchrun --nproc-per-node N scripts/train.py ... [--fsdp-shard]

Flags are generated from ``speculators_b200.train.config.TrainConfig``; ``--config
run.yaml`` layers a YAML file beneath them and ``--dump-config`` prints the resolved
configuration.
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from speculators_b200.train.config import TrainConfig  # noqa: E402
from speculators_b200.train.entrypoint import (  # noqa: E402,F401 - the building blocks stay importable from the script
    _build_from_config_only, build_draft_model, create_transformer_layer_config, load_draft_transformer_layer_config, main,
)

if __name__ == "__main__":
    main(TrainConfig.resolve())
