"""``causal-train`` console entry point."""
from .training.runner import main

__all__ = ["main"]

if __name__ == "__main__":
    raise SystemExit(main())
