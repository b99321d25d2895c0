from dynamis_b200.graph import radius_graph_pbc_cuda  # noqa: F401
