from allie_b200.serve.server import algorithm_test  # noqa: F401
