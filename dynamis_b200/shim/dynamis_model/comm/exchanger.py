from dynamis_b200.exchange import Exchanger, GPUDirectExchanger, PythonNCCLExchanger  # noqa: F401
