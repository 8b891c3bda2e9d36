"""The comparison arm: yinqiwen/lmsf's own kernels, built unmodified, and a step made of them.
Nothing in this folder imports `lmsf_b200`."""
