"""Head-to-head baselines (not product code): cuSPARSE called as the reference calls it."""
