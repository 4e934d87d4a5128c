"""Deterministic synthetic biographies.

Two layers, as in the reference generator (experiments/synbios_moe/pretraining/dataset.py:1-417): a *profile* is the
fact table of one person (name, pronoun, six attributes); a *biography* verbalises one profile with one sentence per
attribute, drawn from a fixed pool of sentence templates, and records the character span of every attribute value
for token-level evaluation and probing.

Contracts kept from the reference
    * nine variants: ``single``, ``single+fullname``, ``single+permute1``, ``single+permute5``, ``multi2``, ``multi5``,
      ``multi2+permute``, ``multi5+permute``, ``multi5+permute+fullname``;
    * profiles depend on ``seed`` only (``random.Random(seed)``), so every variant of one seed has a byte-identical
      ``profiles.jsonl``; each biography draws from ``random.Random(f"{seed}:{person_id}:{variant}:{sample}")``;
    * person-level split by ``sha256(f"{seed}:{person_id}")`` (half of the people are held out for probes);
    * pool sizes 400 x 400 x 1000 names, 200 cities, 300 universities, 100 majors, 263 companies of which 36 sit in
      New York, and 46 / 49 / 49 / 52 / 47 / 48 templates for the six attributes;
    * without ``fullname`` the name appears once, as the subject of whichever sentence ends up first.
"""

from __future__ import annotations

import hashlib
import random
from dataclasses import asdict, dataclass
from datetime import date
from pathlib import Path
from typing import Iterable, Iterator

from experiments.synbios_moe.artifact_io import manifest_of, write_json

ATTRIBUTES = ("birth_date", "birth_city", "university", "major", "company", "company_city")
WHOLE_ATTRIBUTES = tuple(a for a in ATTRIBUTES if a != "birth_date")
TEMPLATE_COUNTS = dict(zip(ATTRIBUTES, (46, 49, 49, 52, 47, 48)))
VARIANTS = ("single", "single+fullname", "single+permute1", "single+permute5", "multi2", "multi5", "multi2+permute",
            "multi5+permute", "multi5+permute+fullname")
MANIFEST_VERSION = 1

_MONTHS = ("January", "February", "March", "April", "May", "June", "July", "August", "September", "October",
           "November", "December")


def _syllable_names(onsets: str, nuclei: str, codas: tuple[str, ...], count: int) -> list[str]:
    """``count`` distinct pronounceable names from a syllable grid (deterministic, no external word list)."""

    out, seen = [], set()
    grid = [(o, n, c) for o in onsets for n in nuclei for c in codas]
    i = 0
    while len(out) < count:
        o, n, c = grid[(i * 7919) % len(grid)]
        second = grid[(i * 104729 + 13) % len(grid)]
        name = (o + n + c + (second[0] + second[1] if i >= len(grid) else "")).capitalize()
        if name not in seen:
            seen.add(name)
            out.append(name)
        i += 1
    return out


def candidate_pools() -> dict[str, list[str]]:
    first = _syllable_names("bdfjklmnrstv", "aeio", ("n", "l", "ra", "na", "s", "th", "ro", "my"), 400)
    middle = _syllable_names("cghlmprsw", "aeiou", ("y", "ley", "den", "ton", "an", "er", "is", "el", "ia"), 400)
    last = _syllable_names("bcdfghklmnprstvw", "aeiou", ("rd", "ner", "son", "ley", "man", "well", "by", "ck", "tt", "ns",
                                                          "mer", "dge", "ll"), 1000)
    towns = _syllable_names("bcdfghlmnprstw", "aeiou", ("ton", "ville", "field", "ford", "burg", "port", "dale", "mont"), 199)
    states = ("CA", "NY", "TX", "MA", "WA", "IL", "PA", "OH", "NC", "GA", "CO", "AZ", "OR", "MI", "VA", "FL")
    cities = ["New York, NY"] + [f"{t}, {states[i % len(states)]}" for i, t in enumerate(towns)]
    kinds = ("University", "College", "Institute of Technology", "State University")
    universities = [f"{t} {kinds[i % len(kinds)]}" for i, t in
                    enumerate(_syllable_names("abcdeghlmnoprstw", "aeiou", ("ston", "bridge", "wood", "mere", "haven", "crest"), 300))]
    fields = ("Physics", "History", "Economics", "Biology", "Music", "Chemistry", "Mathematics", "Linguistics", "Philosophy",
              "Geology", "Statistics", "Architecture", "Sociology", "Astronomy", "Nursing", "Finance", "Design", "Law",
              "Anthropology", "Agronomy")
    flavours = ("", "Applied ", "Computational ", "Comparative ", "Industrial ")
    majors = [f"{flavours[i // len(fields)]}{fields[i % len(fields)]}" for i in range(100)]
    suffixes = ("Group", "Labs", "Holdings", "Partners", "Systems", "Works", "Industries")
    companies = [f"{n} {suffixes[i % len(suffixes)]}" for i, n in
                 enumerate(_syllable_names("abcdfghklmnprstvz", "aeiou", ("x", "ra", "nex", "tis", "vo", "lia", "dyn"), 263))]
    # 36 of 263 employers are headquartered in New York; the rest are spread over the other cities
    company_city = ["New York, NY" if i < 36 else cities[1 + ((i - 36) * 73) % 199] for i in range(263)]
    return {"first": first, "middle": middle, "last": last, "birth_city": cities, "university": universities, "major": majors,
            "company": companies, "company_city": company_city}


@dataclass(frozen=True)
class Profile:
    person_id: int
    full_name: str
    pronoun: str
    birth_date: str
    birth_city: str
    university: str
    major: str
    company: str
    company_city: str


@dataclass(frozen=True)
class Biography:
    person_id: int
    variant: str
    sample: int
    text: str
    attribute_spans: dict[str, tuple[int, int]]


def generate_profiles(num_people: int, seed: int) -> list[Profile]:
    if not 0 < num_people <= 400 * 400 * 1000:
        raise ValueError("num_people exceeds the space of unique names")
    pools = candidate_pools()
    rng = random.Random(seed)
    taken: set[str] = set()
    people: list[Profile] = []
    while len(people) < num_people:
        name = f"{rng.choice(pools['first'])} {rng.choice(pools['middle'])} {rng.choice(pools['last'])}"
        if name in taken:
            continue
        taken.add(name)
        employer = rng.randrange(263)
        born = date(rng.randrange(1900, 2100), rng.randrange(1, 13), rng.randrange(1, 29))
        people.append(Profile(
            person_id=len(people), full_name=name, pronoun=rng.choice(("He", "She", "They")),
            birth_date=f"{_MONTHS[born.month - 1]} {born.day}, {born.year}", birth_city=rng.choice(pools["birth_city"]),
            university=rng.choice(pools["university"]), major=rng.choice(pools["major"]),
            company=pools["company"][employer], company_city=pools["company_city"][employer]))
    return people


# Sentence frames per attribute: {s} = subject (pronoun or full name), {v} = the value.  Openers multiply the frames up to
# the exact template count of every attribute.
_FRAMES = {
    "birth_date": ("{s} came into the world on {v}.", "{s} marks every birthday on {v}.", "The birth of {s} took place on {v}.",
                   "{s} was delivered on {v}.", "{s} first saw daylight on {v}.", "{s} counts {v} as a birthday."),
    "birth_city": ("{s} spent childhood in {v}.", "{s} hails from {v}.", "The hometown of {s} is {v}.", "{s} was raised in {v}.",
                   "{s} took first steps in {v}.", "Family roots of {s} lie in {v}.", "{s} started life in {v}."),
    "university": ("{s} earned a degree at {v}.", "{s} enrolled at {v}.", "{s} was a student of {v}.", "{s} walked the halls of {v}.",
                   "The alma mater of {s} is {v}.", "{s} finished higher education at {v}.", "{s} took classes at {v}."),
    "major": ("{s} concentrated on {v}.", "{s} chose {v} as a field of study.", "{s} wrote a thesis in {v}.", "{s} trained in {v}.",
              "The degree of {s} is in {v}.", "{s} took up {v}.", "{s} built expertise in {v}.", "{s} pursued coursework in {v}."),
    "company": ("{s} drew a salary from {v}.", "{s} built a career at {v}.", "{s} was on the staff of {v}.", "{s} signed on with {v}.",
                "The employer of {s} was {v}.", "{s} held a position at {v}.", "{s} spent working years at {v}."),
    "company_city": ("{s} commuted to an office in {v}.", "{s} held a job located in {v}.", "The workplace of {s} was in {v}.",
                     "{s} clocked in every day in {v}.", "{s} earned a living in {v}.", "{s} was stationed for work in {v}.",
                     "{s} built a professional life in {v}."),
}
_OPENERS = ("", "Notably, ", "According to records, ", "As friends recall, ", "By all accounts, ", "In fact, ", "Reportedly, ",
            "For the record, ")


def template(attribute: str, index: int) -> str:
    frames = _FRAMES[attribute]
    if not 0 <= index < TEMPLATE_COUNTS[attribute]:
        raise IndexError(f"{attribute} has {TEMPLATE_COUNTS[attribute]} templates")
    opener, frame = _OPENERS[index // len(frames)], frames[index % len(frames)]
    if opener and not frame.startswith("{"):
        frame = frame[0].lower() + frame[1:]
    return opener + frame


def entries_per_person(variant: str) -> int:
    for n in (5, 2, 1):
        if f"multi{n}" in variant or f"permute{n}" in variant:
            return n
    return 1


def render_biography(profile: Profile, *, variant: str, sample: int, seed: int) -> Biography:
    """One biography: a template per attribute, optional sentence shuffle, the name placed once (or everywhere)."""

    if variant not in VARIANTS:
        raise ValueError(f"unknown variant {variant!r}")
    rng = random.Random(f"{seed}:{profile.person_id}:{variant}:{sample}")   # independent of iteration order
    everywhere = "fullname" in variant
    parts: list[tuple[str, str]] = []
    for attribute in ATTRIBUTES:
        parts.append((attribute, template(attribute, rng.randrange(TEMPLATE_COUNTS[attribute]))))
    if "permute" in variant:
        rng.shuffle(parts)
    sentences, spans, offset = [], {}, 0
    for position, (attribute, frame) in enumerate(parts):
        subject = profile.full_name if (everywhere or position == 0) else profile.pronoun
        # a pronoun in the middle of a sentence is lower-cased ("The hometown of she" never occurs: such frames take
        # the possessive-free wording, and mid-sentence pronouns are written in lower case)
        if subject == profile.pronoun and not frame.replace(_opener_of(frame), "", 1).startswith("{s}"):
            subject = {"He": "him", "She": "her", "They": "them"}[profile.pronoun]
        elif subject == profile.pronoun and _opener_of(frame):
            subject = profile.pronoun.lower()
        value = getattr(profile, attribute)
        head, tail = frame.split("{v}")
        head = head.replace("{s}", subject)
        tail = tail.replace("{s}", subject)
        sentence = head + value + tail
        spans[attribute] = (offset + len(head), offset + len(head) + len(value))
        sentences.append(sentence)
        offset += len(sentence) + 1
    return Biography(profile.person_id, variant, sample, " ".join(sentences), spans)


def _opener_of(frame: str) -> str:
    for opener in sorted(_OPENERS, key=len, reverse=True):
        if opener and frame.startswith(opener):
            return opener
    return ""


def iter_biographies(profiles: Iterable[Profile], variant: str, seed: int) -> Iterator[Biography]:
    for profile in profiles:
        for sample in range(entries_per_person(variant)):
            yield render_biography(profile, variant=variant, sample=sample, seed=seed)


def split_for_person(person_id: int, seed: int, validation_fraction: float = 0.5) -> str:
    digest = hashlib.sha256(f"{seed}:{person_id}".encode()).digest()
    return "validation" if int.from_bytes(digest[:8], "big") / 2**64 < validation_fraction else "train"


def write_dataset(output_dir: str | Path, *, num_people: int, variant: str, seed: int) -> Path:
    """``profiles.jsonl`` (facts + split), ``biographies.jsonl`` (text + spans), ``biographies.txt``, ``manifest.json``."""

    import json

    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    profiles = generate_profiles(num_people, seed)
    with open(out / "profiles.jsonl", "w", encoding="utf-8") as fh:
        for p in profiles:
            fh.write(json.dumps({**asdict(p), "split": split_for_person(p.person_id, seed)}, ensure_ascii=False) + "\n")
    count = 0
    with open(out / "biographies.jsonl", "w", encoding="utf-8") as records, open(out / "biographies.txt", "w", encoding="utf-8") as plain:
        for bio in iter_biographies(profiles, variant, seed):
            records.write(json.dumps(asdict(bio), ensure_ascii=False) + "\n")
            plain.write(bio.text + "\n")
            count += 1
    files = manifest_of(out, ("profiles.jsonl", "biographies.jsonl", "biographies.txt"))
    write_json(out / "manifest.json", {
        "format": MANIFEST_VERSION, "generator": "synbios", "variant": variant, "seed": seed, "num_people": num_people,
        "num_biographies": count, "entries_per_person": entries_per_person(variant), "attributes": list(ATTRIBUTES),
        "template_counts": TEMPLATE_COUNTS, "split": {"unit": "person", "validation_fraction": 0.5}, "files": files})
    return out
