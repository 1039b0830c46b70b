"""NVIDIA B200 (sm_100a) targets."""
