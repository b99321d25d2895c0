from dynamis_b200.dist_graph_builder import BuildMode, DistBuildGraphResult, DistGraphBuilder  # noqa: F401
