"""Reply parsing and sample-based metrics."""
import pytest

from keys_values_b200.evaluation import metrics as M
from keys_values_b200.evaluation import response_parser as R


def test_normalize_string_response():
    assert R.normalize_string_response("Answer: Paris") == "Paris"
    assert R.normalize_string_response("  answer - label: `42` ") == "42"
    assert R.normalize_string_response("Well, after some thought the answer is: 'blue whale'") == "blue whale"
    assert R.normalize_string_response("In summary the label is 17") == "17"
    assert R.normalize_string_response("</think> Output = yes") == "yes"
    assert R.normalize_string_response(None) == "" and R.normalize_string_response("   ") == ""


def test_extract_numbers_letters_values():
    assert R.extract_numbers("ids 3 > 12 > 1,204 then 7.9 and 2e3.") == ["3", "12", "1204", "7", "2000"]
    assert R.extract_numbers("none here") == ["0"] and R.extract_numbers("x 5 y 6", as_list=False) == "5"
    assert R.extract_numbers("v1.2.3 abc123") == ["0"]  # identifiers and version strings are not numbers
    assert R.extract_choice_letter("I think B is wrong. The correct answer is (C).") == "C"
    assert R.extract_choice_letter("D") == "D" and R.extract_choice_letter("option b, clearly") == "B"
    assert R.extract_choice_letter("no letter", default="?") == "?" and R.extract_choice_letter("E", choices="ABCD") == ""
    assert R.extract_value_token("The special magic uuid for x is: **3f2a9c1e-7b4d-4e8a-9f10**.") == "3f2a9c1e-7b4d-4e8a-9f10"
    assert R.extract_value_token("It mentions 17 first; the number is `4821`") == "4821"
    assert R.extract_value_token("values 12 and 99") == "99" and R.extract_value_token("", default="none") == "none"


def test_match_metrics():
    assert M.exact_match("Answer: Paris", ["paris", "Lyon"]) == 1.0 and M.exact_match("Paris, France", "Paris") == 0.0
    assert M.sub_exact_match("The answer is: the Eiffel Tower in Paris", ["eiffel tower"]) == 1.0
    assert M.sub_exact_match("Eifel towr", "Eiffel Tower") == 0.0 and M.sub_exact_match("Eifel towr", "Eiffel Tower", threshold=0.8) == 1.0
    assert M.sub_exact_similarity("tower eiffel", "Eiffel Tower") == 1.0
    assert M.rouge_n_f1("the cat sat", ["a cat sat down"], n=1) == pytest.approx(2 * (2 / 2) * (2 / 3) / ((2 / 2) + (2 / 3)))
    assert M.multiple_choice_letter("The correct answer is (B)", "B") == 1.0 and M.multiple_choice_letter("A or maybe C", "(A)") == 0.0
    assert M.synthetic_value_match("The special magic number for k is 4821.", ["4821"]) == 1.0
    assert M.synthetic_value_match("they are 11 and 22", ["11", "22"]) == 1.0 and M.synthetic_value_match("it is 12", ["13"]) == 0.0


def test_ndcg_ranked_numbers():
    assert M.ndcg_at_10_ranked_numbers(["3", "1", "2"], ["3", "1", "2"]) == pytest.approx(1.0)
    assert M.ndcg_at_10_ranked_numbers(["03", "1.0", "2"], ["3", "1", "2"]) == pytest.approx(1.0)  # numeric identity
    worse = M.ndcg_at_10_ranked_numbers(["2", "1", "3"], ["3", "1", "2"])
    assert 0.0 < worse < 1.0
    assert M.ndcg_at_10_ranked_numbers(["3", "3", "3"], ["3", "1", "2"]) < M.ndcg_at_10_ranked_numbers(["3", "1"], ["3", "1", "2"])
    assert M.ndcg_at_10_ranked_numbers([], ["1"]) == 0.0 and M.ndcg_at_10_ranked_numbers(["x"], []) == 0.0
    assert M.METRICS["ndcg_at_10"]("Ranking: 3 > 1 > 2", "3 > 1 > 2") == pytest.approx(1.0)
    assert M.HELMET_TASK_METRIC["nq"] == "sub_exact_match" and M.HELMET_TASK_METRIC["ms_macro"] == "ndcg_at_10"
