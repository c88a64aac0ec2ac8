from allie_b200.models import Model, initialize_model  # noqa: F401
from allie_b200.models.oracle import CausalLMWithControlToken, CausalLMWithRegressionHead  # noqa: F401
