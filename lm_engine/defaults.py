"""Prompt templates: the dataset example is substituted for the placeholders."""

INPUT_FORMAT = "__input__"
OUTPUT_FORMAT = "__output__"
