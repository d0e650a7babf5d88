"""Process-wide seeding (reference: seed.py:6-11)."""
import random

import numpy as np
import torch


def set_seed(seed: int) -> None:
    """Seed numpy, ``random``, torch CPU and every CUDA generator with ``seed``.

    Compressed reducers in this library do not depend on these generators: their
    rounding noise and index sets come from the counter-based Philox streams in
    ``ops.philox``, so re-seeding here never correlates ranks' rounding noise.
    """
    np.random.seed(seed)
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
