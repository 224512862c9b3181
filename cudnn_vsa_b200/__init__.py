"""B200-native packed video-sparse-attention (VSA) hot path."""
