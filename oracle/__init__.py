"""CPU oracle for the dense training step (TEST INFRASTRUCTURE ONLY).

Nothing in the product package may import this directory: only the tests, the
smoke entry and the bench's CPU-baseline legs use it, and only as the checker
or as the timed CPU arm.  The product path is CUDA and fails loudly when its
extension is missing.

Pinning: `oracle.model` with `Arch.reference()` is checked against the
reference's own `tests/reference.py` (imported in the development container)
through the golden vectors under `tests/golden/`, and the optimizer / schedule
restatements are checked against torch.optim (AdamW, Muon, OneCycleLR), the
same expected-value side the reference's `tests/verify.py` uses.
"""
