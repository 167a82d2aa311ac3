"""Convert a checkpoint of this engine into a Hugging Face architecture."""

from argparse import ArgumentParser

from ..hf_models import export_to_huggingface


def main() -> None:
    parser = ArgumentParser(description=__doc__)
    parser.add_argument("--model", required=True, help="directory with config.json and safetensors of this engine")
    parser.add_argument("--save-path", required=True)
    parser.add_argument("--model-type", required=True,
                        choices=["llama", "granite", "granitemoe", "granitemoeshared", "granitemoehybrid", "gpt_bigcode"])
    args = parser.parse_args()
    export_to_huggingface(args.model, args.save_path, args.model_type)


if __name__ == "__main__":
    main()
