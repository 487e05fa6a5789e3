"""B200-native UVU TensorProductConv hot path (sm_100a CUDA behind a C-ABI) with the reference's Python surface."""
