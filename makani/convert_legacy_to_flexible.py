"""`python -m makani.convert_legacy_to_flexible`: the upstream command name for `python -m makani_b200.convert_legacy_to_flexible` (same flags)."""

from makani_b200.convert_legacy_to_flexible import main

if __name__ == "__main__":
    main()
