"""B200-native SAM image-encoder hot path behind the segment_anything_fast API."""
