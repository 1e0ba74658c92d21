"""`python testcon.py ...`: the concurrent serving test from the repository root (same arguments as
`python -m fastcache_b200.serving.testcon`)."""
from fastcache_b200.serving.testcon import main

if __name__ == "__main__":
    main()
