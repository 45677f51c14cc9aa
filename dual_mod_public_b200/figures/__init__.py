"""Figure renderers for the formal-language, TinyStories and fixed-point experiments (dependency-free SVG)."""
