from dynamis_b200.exchange import FeaturePushToExchange  # noqa: F401
