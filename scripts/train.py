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
from speculators_b200.train.entrypoint import main  # noqa: E402

if __name__ == "__main__":
    main(TrainConfig.resolve())
