"""Python wrappers around the native sm_100a kernels."""
