"""Command-line entry points: RL training, evaluation-only, stand-alone rollout serving, SFT."""
