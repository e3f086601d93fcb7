"""Small helpers: environment report, training-log line format."""
