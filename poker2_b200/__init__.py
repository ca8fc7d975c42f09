"""poker2_b200: hand-written sm_100a kernels for ReBeL subgame solving (hand ranking,
river showdown, fused CFR iteration), behind a C ABI with Python host code that mirrors
the call signatures of the upstream P2 search modules."""

__all__ = ["rules", "showdown"]
