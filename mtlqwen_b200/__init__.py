"""B200-native forward step for the MTLQwen engine API (sm_100a CUDA behind a C ABI)."""
