"""Dataset recipes selectable from a CLI config (`data_module: tunix_b200.cli.recipes.<name>`)."""
