"""Export of trained weights to inference runtimes."""
