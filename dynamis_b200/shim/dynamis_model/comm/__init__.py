from dynamis_model.comm import drift_flags  # noqa: F401
