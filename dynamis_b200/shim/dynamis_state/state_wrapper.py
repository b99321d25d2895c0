from dynamis_b200.dist_env import TorchDistEnv  # noqa: F401
