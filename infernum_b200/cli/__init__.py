"""Command-line programs: generate, bench, trace replay."""
