"""CPU oracle of the ConvNN-Attention forward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this folder.  Allowed importers: ``tests/``, the
smoke entry, and the CPU-baseline legs of ``bench.py`` (as the thing timed on the host
cores, never as the GPU path).  Parity status: pinned against outputs of the unmodified
reference (see ``pin_against_reference.py`` and ``tests/golden/``).
"""
