"""The factor-preparation names of the reference's ``gptq_2d_reference.py`` (``ldl_of_inverse``,
``feedback_factors``, :41-66), served by the CUDA pipeline of ``kron_factors``.  The paper-listing algorithms of that
file are test oracles of the reference and are not part of this package."""
from kron_factors import feedback_factors, gptq_d_sided, ldl_of_inverse  # noqa: F401

alg4 = gptq_d_sided  # the reference's name for N-factor rounding (gptq_2d_reference.py:270)
