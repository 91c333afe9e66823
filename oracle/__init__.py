"""CPU oracle of reflex-infer's paged-KV attention path. TEST INFRASTRUCTURE ONLY.

Nothing in the product (``reflex-infer_b200/``) imports this package; it is used by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline and
reference legs, always as the checker or the thing the GPU path is compared against,
never as the implementation.

Pinning: every function here is checked in ``tests/test_oracle_golden.py`` against
vectors produced by importing the reference's own torch path (``tests/golden/make_golden.py``).
The arithmetic lives in PyTorch's CPU kernels, as it does in the reference
(``torch>=2.5`` per its ``pyproject.toml:27-31``); the fixtures record the torch version
that produced them.
"""
from .torch_oracle import *  # noqa: F401,F403
