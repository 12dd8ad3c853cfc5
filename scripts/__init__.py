"""Evidence tooling: aggregate measurement records, recompute cohort statistics, render tables, probe gradient bounds."""
