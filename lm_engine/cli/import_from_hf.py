"""Convert a Hugging Face checkpoint (llama, granite, granitemoe, granitemoeshared, granitemoehybrid, gpt_bigcode) into
this engine's format."""

from argparse import ArgumentParser

from ..hf_models import import_from_huggingface


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--model", required=True, help="local directory or hub name of the Hugging Face model")
    parser.add_argument("--save-path", required=True)
    args = parser.parse_args()
    import_from_huggingface(args.model, args.save_path)


if __name__ == "__main__":
    main()
