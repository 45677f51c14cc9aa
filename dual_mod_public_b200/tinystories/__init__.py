"""TinyStories ablation trainer (exact sequential scan, torch DDP)."""
