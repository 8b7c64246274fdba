"""iris_b200: a Blackwell-native symmetric-memory multi-GPU framework (work in progress)."""
