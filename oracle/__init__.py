"""CPU restatement of the aimet_torch quantization-simulation hot path.

TEST INFRASTRUCTURE ONLY.  These modules restate, op by op with PyTorch CPU tensor arithmetic, what
the reference computes, so that the CUDA kernels can be checked against them on a machine where
the reference itself is not installed.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this package; the product
package ``aimet_b200`` never does and has no CPU path of its own.

Parity pin: every function here is checked bit-for-bit against fixtures under ``tests/golden/``
that were produced by running the reference's own Python code (``tests/golden/make_golden.py``),
including the known-answer vector sets of the reference's ``test_backend.py``.

Citations give paths relative to ``TrainingExtensions/torch/src/python/aimet_torch/``.
"""
