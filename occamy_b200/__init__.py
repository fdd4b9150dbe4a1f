"""occamy_b200 -- B200-native operator runtime behind the Occamy DNN dialect's C ABI.

``runtime``  ctypes binding of liboccamy_dnn.so (the product: sm_100a kernels + arena)
``replay``   program builder / pool planner / replayer (stand-in for a compiled model)
``graphs``   the benchmark graphs with seeded synthetic weights
``build``    in-tree nvcc build of the native libraries
"""
__all__ = ["runtime", "replay", "graphs", "build"]
