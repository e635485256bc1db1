"""``from fla.ops.gated_delta_rule import chunk_gated_delta_rule`` as the reference writes it."""
from atma_b200.gated_delta import chunk_gated_delta_rule  # noqa: F401
