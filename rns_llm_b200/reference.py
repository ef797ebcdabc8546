"""Names of the reference's ``rns_llm.reference`` module that are host-side
constants, re-exported so that ``from rns_llm_b200.reference import
choose_moduli_for_dot`` works like its reference counterpart.  The NumPy
encoders/decoders of that module are CPU arithmetic and are not part of this
package."""
from .moduli import (  # noqa: F401
    DENSE_COPRIME_MODULI,
    HARDWARE_FRIENDLY_MODULI,
    LARGE_PRIME_MODULI,
    SMALL_PRIME_MODULI,
    candidates_for_strategy,
    choose_moduli_for_dot,
    compact_byte_mod_lut,
    crt_constants,
    dot_product_bound,
    garner_pairwise_inverses,
    moduli_cost_model,
    validate_moduli,
)
