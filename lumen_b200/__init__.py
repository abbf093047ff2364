"""lumen_b200: a B200-native CUDA execution backend for lumen's compiled graphs."""
