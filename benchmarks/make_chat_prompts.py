"""Generator of the chat-style prompt set ``benchmarks/chat_prompts_500.csv``.

    python benchmarks/make_chat_prompts.py [--num 500] [--seed 0] [--out benchmarks/chat_prompts_500.csv]

The reference measures serving throughput on a sample of real user conversations (benchmarks/share_gpt_500.csv there);
conversations cannot be shipped here, so this script composes first turns of the same kinds (a bare question, a
request with pasted material, a continuation that quotes an earlier answer, code with an error message, a table to
rework) with a long-tailed length distribution: most prompts are a line or two, a few run to several thousand
characters, as in chat traffic. The text is assembled from word lists below with a seeded generator, so the file can
be rebuilt bit for bit; one column named ``query``, read by ``benchmark_throughput.py --input_csv``.
"""
import argparse
import csv
import math
import os
import random

TOPICS = [
    "a weekly meal plan for two", "the causes of the French Revolution", "a binary heap", "index funds", "sourdough bread",
    "the water cycle", "a REST API for a library", "tidal locking of moons", "a marathon training block", "compound interest",
    "version control branching", "the rules of cricket", "a small vegetable garden", "SQL window functions", "the Doppler effect",
    "a cover letter for a nursing job", "a retrospective meeting", "photosynthesis", "a unit test suite", "the history of the bicycle",
    "a budget for a school trip", "regular expressions", "plate tectonics", "a product launch email", "a chess opening for beginners",
    "sleep hygiene", "a command-line to-do list", "the periodic table", "a wedding toast", "container orchestration",
    "the Silk Road", "a job interview for a data analyst", "knitting a scarf", "public-key cryptography", "a haiku about rain",
    "noise-cancelling headphones", "an onboarding checklist", "Bayes' theorem", "a bedtime story about a fox", "bicycle gear ratios",
]
ASKS = [
    "Can you explain {t} to someone who has never heard of it?", "Give me a step-by-step plan for {t}.",
    "What are the three most common mistakes people make with {t}?", "Write a short introduction to {t} for a newsletter.",
    "Summarise what matters most about {t} in five bullet points.", "I have ten minutes to prepare a talk on {t}. What do I say?",
    "Compare two ways of approaching {t} and say which you would pick.", "Draft an outline of a blog post about {t}.",
    "Ask me five questions that would show whether I understand {t}.", "Rewrite my notes on {t} so that a ten-year-old could follow them.",
]
FOLLOW_UPS = [
    "Make it shorter.", "Now make the tone more formal.", "Add a concrete example.", "Turn that into a table.",
    "Give me the same thing as a checklist.", "What would you change for a team of five?", "Explain the second point again, more slowly.",
]
SUBJECTS = ["the team", "our supplier", "the committee", "my manager", "the client", "the city council", "the school", "the lab", "the editor", "the landlord"]
VERBS = ["postponed", "approved", "questioned", "rewrote", "measured", "rejected", "outlined", "shortened", "doubled", "reviewed"]
OBJECTS = ["the quarterly budget", "the delivery schedule", "the safety report", "the second draft", "the test results", "the floor plan",
           "the hiring plan", "the poll results", "the maintenance contract", "the release notes"]
TAILS = ["after a long discussion", "without telling anyone", "for the third time this year", "because the figures did not add up",
         "and asked for a summary by Friday", "although nobody had objected", "so the deadline moved by two weeks", "which surprised everyone",
         "and nobody knows why", "before the holidays"]
CODE_LANGS = [("Python", "def total(items):\n    s = 0\n    for i in range(len(items) + 1):\n        s += items[i].price\n    return s", "IndexError: list index out of range"),
              ("JavaScript", "async function load(id) {\n  const res = fetch('/api/items/' + id);\n  return res.json();\n}", "TypeError: res.json is not a function"),
              ("SQL", "SELECT customer, SUM(amount)\nFROM orders\nWHERE SUM(amount) > 100\nGROUP BY customer;", "ERROR: aggregate functions are not allowed in WHERE"),
              ("C", "char *copy(const char *s) {\n  char buf[16];\n  strcpy(buf, s);\n  return buf;\n}", "warning: function returns address of local variable"),
              ("Go", "func worker(ch chan int) {\n  for v := range ch {\n    fmt.Println(v)\n  }\n}\nfunc main() {\n  ch := make(chan int)\n  ch <- 1\n  go worker(ch)\n}", "fatal error: all goroutines are asleep - deadlock!")]
COLUMNS = ["Task", "Owner", "Due", "Status", "Risk", "Cost", "Notes"]


def sentence(rng):
    return f"{rng.choice(SUBJECTS).capitalize()} {rng.choice(VERBS)} {rng.choice(OBJECTS)} {rng.choice(TAILS)}."


def paragraph(rng, n):
    return " ".join(sentence(rng) for _ in range(n))


def pasted_material(rng, sentences):
    """Paragraphs of filler prose: the material a user pastes under a request."""
    paras, left = [], sentences
    while left > 0:
        n = min(left, rng.randint(2, 7))
        paras.append(paragraph(rng, n))
        left -= n
    return "\n\n".join(paras)


def table(rng, rows):
    cols = rng.sample(COLUMNS, rng.randint(3, 5))
    lines = ["| " + " | ".join(cols) + " |", "|" + " --- |" * len(cols)]
    for _ in range(rows):
        lines.append("| " + " | ".join(rng.choice(OBJECTS + SUBJECTS + TAILS) for _ in cols) + " |")
    return "\n".join(lines)


def one_prompt(rng):
    # long-tailed amount of attached material: log-normal number of sentences, most draws give none or a few
    amount = int(math.exp(rng.gauss(1.2, 1.3)))
    kind = rng.random()
    topic = rng.choice(TOPICS)
    ask = rng.choice(ASKS).format(t=topic)
    if kind < 0.35 or amount == 0:
        return ask if rng.random() < 0.7 else ask[0].lower() + ask[1:].rstrip("?.")          # bare, sometimes sloppy
    if kind < 0.60:
        lead = rng.choice(["Summarise the following for a colleague who missed the meeting:", "Proofread this and list what you changed:",
                           "Translate the key points of this into plain language:", "Write a reply to this message, polite but firm:"])
        return f"{lead}\n\n{pasted_material(rng, amount)}"
    if kind < 0.75:
        earlier = pasted_material(rng, max(2, amount // 2))
        return f"Earlier you wrote:\n\n\"{earlier}\"\n\n{rng.choice(FOLLOW_UPS)} {ask}"
    if kind < 0.90:
        lang, code, err = rng.choice(CODE_LANGS)
        extra = f"\n\nContext: {paragraph(rng, min(amount, 6))}" if amount > 3 else ""
        return f"This {lang} code fails with `{err}`. What is wrong and how do I fix it?\n\n```\n{code}\n```{extra}"
    return f"Sort this table by its {rng.choice(['first', 'second', 'last'])} column, merge rows that say the same thing and point out anything that looks inconsistent.\n\n{table(rng, min(3 + amount, 40))}"


def build(num, seed):
    rng = random.Random(seed)
    return [one_prompt(rng) for _ in range(num)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--num", type=int, default=500)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "chat_prompts_500.csv"))
    args = ap.parse_args()
    prompts = build(args.num, args.seed)
    with open(args.out, "w", encoding="utf-8", newline="") as f:
        w = csv.writer(f)
        w.writerow(["query"])
        for p in prompts:
            w.writerow([p])
    lens = sorted(len(p) for p in prompts)
    print(f"{len(prompts)} prompts -> {args.out}; characters: median {lens[len(lens) // 2]}, p90 {lens[int(len(lens) * 0.9)]}, max {lens[-1]}")


if __name__ == "__main__":
    main()
