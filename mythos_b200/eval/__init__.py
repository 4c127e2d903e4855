"""Evaluation (the reference's src/eval.cpp): sliding-window perplexity, next-token accuracy,
classification precision/recall/F1, BLEU, ROUGE-L, multiple-choice scoring."""
from .metrics import (ModelEvaluator, compute_bleu, compute_rouge_l, eval_accuracy, eval_classification,  # noqa: F401
                      eval_multiple_choice, eval_perplexity)
