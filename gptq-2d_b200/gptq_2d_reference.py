"""The names of the reference's ``gptq_2d_reference.py`` that belong to the rounding path: the factor preparation
(``ldl_of_inverse``, ``feedback_factors``, :41-66) and N-factor rounding (``alg4``, :269-294), served by the CUDA
pipelines of ``kron_factors``.  The other paper-listing algorithms of that file are test oracles of the reference and are
not part of this package."""
from kron_factors import alg4, feedback_factors, gptq_d_sided, ldl_of_inverse  # noqa: F401
