"""Testing toolkit shipped with the package: toy models, a fixed-vocabulary tokenizer, tree comparisons and a base
class for LoRA export tests, for tests written against this framework."""
